"""Grouped (ragged-M) FP8 GEMM behind the reference's gmm(a, b, batch_sizes, trans_b) signature
(op/grouped_gemm/cudaop_grouped_gemm/ops.py:76-83; its test splits tokens into uneven groups, zero-sized ones included:
op/grouped_gemm/test_grouped_gemm.py).  Every group is checked against the oracle GEMM on the same quantised bytes."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


def _case(sizes, N, K, seed):
    rng = np.random.default_rng(seed)
    T, E = int(sum(sizes)), len(sizes)
    a = oracle.encode_e4m3(rng.standard_normal((T, K), dtype=np.float32))
    b = oracle.encode_e4m3(rng.standard_normal((E, N, K), dtype=np.float32))
    sa = rng.uniform(0.5, 2.0, T).astype(np.float32)
    sb = rng.uniform(0.001, 0.01, (E, N)).astype(np.float32)
    return a, sa, b, sb


def _check(out, a, sa, b, sb, sizes, K, what):
    off = 0
    for e, n in enumerate(sizes):
        if n == 0:
            continue
        ref = oracle.gemm_f32(oracle.decode_e4m3(a[off:off + n]), oracle.decode_e4m3(b[e]), threads=CORES) * (sa[off:off + n, None] * sb[e][None, :])
        assert_bar(bf16_to_f32(out[off:off + n]), ref, K, f"{what} group {e}")
        off += n


@pytest.mark.parametrize("sizes,N,K", [([128, 128], 256, 128), ([5, 0, 300, 129, 1, 0, 77], 520, 272), ([0, 0, 64], 8, 16),
                                       ([1000, 24], 1000, 1040), ([3] * 40, 384, 512), ([700, 0, 1348], 2048, 1024)])
@pytest.mark.parametrize("where", ["cpu", "cuda"])
def test_groups_against_the_oracle(sizes, N, K, where):
    import cudaop_b200 as ops
    a, sa, b, sb = _case(sizes, N, K, seed=len(sizes) + N + K)
    bs = torch.tensor(sizes, dtype=torch.int64, device=where)
    out = ops.gmm_fp8(dev(a), dev(sa), dev(b), dev(sb), bs)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert out.shape == (sum(sizes), N) and out.dtype == torch.bfloat16
    _check(out, a, sa, b, sb, sizes, K, "gmm_fp8")


def test_rows_outside_every_group_stay_zero_and_sizes_are_clamped():
    import cudaop_b200 as ops
    sizes, N, K = [100, 50], 128, 128
    a, sa, b, sb = _case([200], N, K, seed=3)                 # 200 tokens, groups cover 150
    b = np.concatenate([b, b], 0); sb = np.concatenate([sb, sb], 0)
    out = ops.gmm_fp8(dev(a), dev(sa), dev(b), dev(sb), torch.tensor(sizes))
    torch.cuda.synchronize()
    assert (out[150:] == 0).all()
    _check(out, a, sa, b, sb, sizes, K, "partial cover")
    # a batch size that runs past the last token is cut off there
    out = ops.gmm_fp8(dev(a), dev(sa), dev(b), dev(sb), torch.tensor([150, 500]))
    torch.cuda.synchronize()
    _check(out, a, sa, b, sb, [150, 50], K, "clamped")
    assert ops.status() == 0


@pytest.mark.parametrize("trans_b", [False, True])
def test_reference_signature_on_bf16_tensors(trans_b):
    """gmm(a, b, batch_sizes, trans_b) on bf16 inputs: activations quantised per token, weights per output channel;
    compared with the same arithmetic done by the oracle (quantisers bit-exact, then the grouped product)."""
    import cudaop_b200 as ops
    sizes, N, K = [130, 0, 61, 200], 192, 256
    rng = np.random.default_rng(17)
    T, E = sum(sizes), len(sizes)
    a = oracle.encode_bf16(rng.standard_normal((T, K), dtype=np.float32))
    w = oracle.encode_bf16(rng.standard_normal((E, N, K), dtype=np.float32) * 0.05)      # [E, N, K]
    a_t = dev(a, torch.bfloat16)
    w_t = dev(w, torch.bfloat16)
    b_arg = w_t if trans_b else w_t.transpose(1, 2).contiguous()                          # reference layout [E, K, N]
    out = ops.gmm(a_t, b_arg, torch.tensor(sizes), trans_b=trans_b)
    weights = ops.GroupedFP8Weights(b_arg, trans_b)
    out2 = ops.gmm(a_t, weights, torch.tensor(sizes))
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    aq, sa = oracle.quant_rows_e4m3(oracle.decode_bf16(a))
    wq, sw = oracle.quant_rows_e4m3(oracle.decode_bf16(w).reshape(E * N, K))
    _check(out, aq, sa, wq.reshape(E, N, K), sw.reshape(E, N), sizes, K, "gmm")
    # and it is close to the unquantised grouped product (information: E4M3 quantisation error, a few percent)
    off = 0
    for e, n in enumerate(sizes):
        if n:
            ref = oracle.decode_bf16(a[off:off + n]) @ oracle.decode_bf16(w[e]).T
            rel = np.linalg.norm(bf16_to_f32(out[off:off + n]) - ref) / np.linalg.norm(ref)
            assert rel < 0.08, rel
        off += n


def test_argument_errors():
    import cudaop_b200 as ops
    a = torch.zeros((64, 128), dtype=torch.uint8, device="cuda"); sa = torch.ones(64, device="cuda")
    b = torch.zeros((2, 32, 128), dtype=torch.uint8, device="cuda"); sb = torch.ones((2, 32), device="cuda")
    with pytest.raises(ValueError):
        ops.gmm_fp8(a, sa, b, sb, torch.tensor([32, 32], dtype=torch.int32))          # batch_sizes must be int64
    with pytest.raises(ValueError):
        ops.gmm_fp8(a, sa, b, sb, torch.tensor([64]))                                  # one entry per expert
    with pytest.raises(ValueError):
        ops.gmm_fp8(a, sa, b[:, :, :64].contiguous(), sb, torch.tensor([32, 32]))      # K mismatch
    torch.cuda.synchronize()
