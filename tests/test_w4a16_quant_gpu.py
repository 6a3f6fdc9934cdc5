"""Parity of the INT4 weight-only decode GEMM and of the activation quantiser."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[(0, 0), (3, 1), (4, 0), (1, 0), (2, 0)], ids=["by_m", "gemv_pdl", "gemv_regs", "tcgen05", "warp_mma"],
                autouse=True)
def impl(request):
    """Every implementation behind b200q_gemm_w4a16: the default (streaming CUDA-core GEMV for one token, warp-MMA
    kernel above), the GEMV for up to four tokens with programmatic dependent launch, its form with the
    weights in registers, the tcgen05 kernel, the warp-MMA kernel for every M."""
    import cudaop_b200 as ops
    ops.lib().b200q_w4a16_set_impl(request.param[0])
    ops.lib().b200q_w4a16_set_pdl(request.param[1])
    yield request.param
    ops.lib().b200q_w4a16_set_impl(0)
    ops.lib().b200q_w4a16_set_pdl(0)


def _w4_ref(xb, wq, s, group=128):
    return oracle.gemm_f32(oracle.decode_bf16(xb), oracle.dequant_w4(wq, s, group), threads=CORES)


@pytest.mark.parametrize("M", [1, 2, 4, 16])
def test_config_decode_4096(M):
    # M in {1,16}, N=K=4096, ints in [-8,7], group 128 fp16 scales U(0.005,0.02), bf16 N(0,1) activations
    import cudaop_b200 as ops
    xb, wq, s = oracle.make_w4a16_case(M, 4096, 4096, seed=0)
    out = ops.gemm_w4a16(dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16))
    torch.cuda.synchronize()
    rep = assert_bar(bf16_to_f32(out), _w4_ref(xb, wq, s), 4096, f"w4a16 M={M}")
    print("w4a16", M, rep)


def test_int4_known_answer_is_exact():
    # op/test/arch_primitives/ptx_mma_integer.cu:61-74: coordinate-dependent S4 values, exact result
    import cudaop_b200 as ops
    M, N, K = 16, 40, 256
    W = np.array([[((n * 5 + k * 3 + 2) % 15) - 7 for k in range(K)] for n in range(N)], np.int8)
    X = np.array([[((m * 2 + k * 7 + 4) % 15) - 7 for k in range(K)] for m in range(M)], np.float32)
    s = np.full((N, K // 128), 1.0, np.float32)
    s[:, 1] = 0.5
    out = ops.gemm_w4a16(dev(oracle.encode_bf16(X), torch.bfloat16), dev(oracle.pack_s4(W)),
                         dev(oracle.encode_f16(s), torch.float16))
    torch.cuda.synchronize()
    want = X[:, :128] @ W[:, :128].T.astype(np.float32) + 0.5 * (X[:, 128:] @ W[:, 128:].T.astype(np.float32))
    assert np.array_equal(bf16_to_f32(out), oracle.decode_bf16(oracle.encode_bf16(want)))


@pytest.mark.parametrize("shape", [(1, 32, 128), (3, 33, 256), (16, 100, 1024), (17, 64, 384), (40, 4096, 2048),
                                   (2, 11008, 4096), (1, 4096, 11008), (4, 130, 9344), (3, 7, 1152)])
def test_ragged_shapes(shape):
    import cudaop_b200 as ops
    M, N, K = shape
    xb, wq, s = oracle.make_w4a16_case(M, N, K, seed=M * 7 + N)
    out = ops.gemm_w4a16(dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16))
    torch.cuda.synchronize()
    assert_bar(bf16_to_f32(out), _w4_ref(xb, wq, s), K, str(shape))


@pytest.mark.parametrize("shape", [(4096, 4096), (100, 2048), (1000, 8192), (4099, 4096), (37, 16384), (28672, 4096),
                                   (8, 6144)])
@pytest.mark.parametrize("pdl", [0, 1])
def test_one_token_streaming_form(shape, pdl, impl):
    """The streaming GEMV (whole weight block of a CTA prefetched by bulk copies, K a multiple of 2048 up to 16384):
    ragged row counts, several CTAs per SM, scales loaded by copy or by threads, with and without programmatic
    dependent launch, three calls in a row on different weights."""
    import cudaop_b200 as ops
    if impl != (0, 0):
        pytest.skip("selects its own implementation")
    N, K = shape
    ops.lib().b200q_w4a16_set_impl(5)
    ops.lib().b200q_w4a16_set_pdl(pdl)
    cases = [oracle.make_w4a16_case(1, N, K, seed=N + K + i) for i in range(2 if N > 8000 else 3)]
    devs = [(dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16)) for xb, wq, s in cases]
    outs = [ops.gemm_w4a16(*d) for d in devs]              # back to back on one stream
    torch.cuda.synchronize()
    assert ops.status() == 0
    for (xb, wq, s), out in zip(cases, outs):
        assert_bar(bf16_to_f32(out), _w4_ref(xb, wq, s), K, f"stream {shape} pdl={pdl}")


def test_one_token_streaming_form_propagates_non_finite_activations(impl):
    import cudaop_b200 as ops
    if impl != (0, 0):
        pytest.skip("selects its own implementation")
    xb, wq, s = oracle.make_w4a16_case(1, 64, 2048, seed=9)
    x = oracle.decode_bf16(xb).copy(); x[0, 5] = np.inf
    ops.lib().b200q_w4a16_set_impl(5)
    out = ops.gemm_w4a16(dev(oracle.encode_bf16(x), torch.bfloat16), dev(wq), dev(s, torch.float16))
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()                  # Inf * 0-weight terms make the reference NaN as well


@pytest.mark.parametrize("shape", [(17, 128, 128), (64, 256, 256), (200, 130, 1152), (129, 1000, 384), (512, 4096, 4096),
                                   (300, 72, 16384), (2, 40, 256)])
@pytest.mark.parametrize("form", [6, 7, 8])
def test_prefill_form(shape, form, impl):
    """The tcgen05 prefill kernel (integer weights on the tensor core, the group's scale applied to its fp32 partial
    sum), in its forms (6: the converters leave the offset 136 in and sixteen rows of ones take it out; 7: the
    converters subtract it; 8: the converted weights are the tensor-memory operand and the product is computed
    transposed): ragged token and row counts, one to 128 groups; every output against the oracle."""
    import cudaop_b200 as ops
    if impl != (0, 0):
        pytest.skip("selects its own implementation")
    M, N, K = shape
    ops.lib().b200q_w4a16_set_impl(form)
    xb, wq, s = oracle.make_w4a16_case(M, N, K, seed=M + N + K)
    out = ops.gemm_w4a16(dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16))
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert_bar(bf16_to_f32(out), _w4_ref(xb, wq, s), K, f"prefill {shape}")


def test_prefill_known_answer_and_default_dispatch(impl):
    """Coordinate-dependent S4 values (op/test/arch_primitives/ptx_mma_integer.cu:61-74) with scales 1 and 0.5 per
    group: every product and sum is exact, so the output equals bf16(expected) bit for bit; 80 tokens go to the
    prefill kernel by default."""
    import cudaop_b200 as ops
    if impl != (0, 0):
        pytest.skip("default dispatch only")
    M, N, K = 80, 40, 256
    W = np.array([[((n * 5 + k * 3 + 2) % 15) - 7 for k in range(K)] for n in range(N)], np.int8)
    X = np.array([[((m * 2 + k * 7 + 4) % 15) - 7 for k in range(K)] for m in range(M)], np.float32)
    s = np.full((N, K // 128), 1.0, np.float32); s[:, 1] = 0.5
    out = ops.gemm_w4a16(dev(oracle.encode_bf16(X), torch.bfloat16), dev(oracle.pack_s4(W)), dev(oracle.encode_f16(s), torch.float16))
    torch.cuda.synchronize()
    want = X[:, :128] @ W[:, :128].T.astype(np.float32) + 0.5 * (X[:, 128:] @ W[:, 128:].T.astype(np.float32))
    assert np.array_equal(bf16_to_f32(out), oracle.decode_bf16(oracle.encode_bf16(want)))


def test_prefill_full_size_sampled_rows(impl):
    import cudaop_b200 as ops
    if impl != (0, 0):
        pytest.skip("default dispatch only")
    M, N, K = 4096, 4096, 4096
    xb, wq, s = oracle.make_w4a16_case(M, N, K, seed=77)
    out = ops.gemm_w4a16(dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16))
    torch.cuda.synchronize()
    assert ops.status() == 0
    rows = np.random.default_rng(1).choice(M, 256, replace=False)
    ref = oracle.gemm_f32(oracle.decode_bf16(xb[rows]), oracle.dequant_w4(wq, s), threads=CORES)
    assert_bar(bf16_to_f32(out[torch.from_numpy(rows).cuda()]), ref, K, "prefill 4096^3 rows")


def test_w4a16_is_deterministic():
    import cudaop_b200 as ops
    xb, wq, s = oracle.make_w4a16_case(16, 4096, 4096, seed=5)
    x, w, sc = dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16)
    a = ops.gemm_w4a16(x, w, sc); b = ops.gemm_w4a16(x, w, sc)
    assert torch.equal(a, b)


def test_w4a16_argument_errors():
    import cudaop_b200 as ops
    L = ops.lib()
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(32, 128, dtype=torch.uint8, device="cuda")
    s = torch.zeros(32, 2, dtype=torch.float16, device="cuda")
    y = torch.zeros(1, 32, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert L.b200q_gemm_w4a16(x.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(), 1, 32, 256, 64, st) == 1
    assert L.b200q_gemm_w4a16(x.data_ptr(), None, s.data_ptr(), y.data_ptr(), 1, 32, 256, 128, st) == 1
    assert L.b200q_gemm_w4a16(x.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(), 1, 32, 200, 128, st) == 1
    assert L.b200q_gemm_w4a16(x.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(), 1, 32, 256, 128, st) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("shape", [(1, 8), (7, 64), (300, 8192), (64, 28672), (33, 3584)])
def test_activation_quantiser_is_bit_exact(shape):
    import cudaop_b200 as ops
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    xb = oracle.encode_bf16(rng.standard_normal((rows, cols), dtype=np.float32) * rng.uniform(0.01, 30, (rows, 1)).astype(np.float32))
    if rows > 2:
        xb[2] = 0          # an all-zero row: scale 1, all zeros
    q, s = ops.quant_rows_e4m3(dev(xb, torch.bfloat16))
    torch.cuda.synchronize()
    q_ref, s_ref = oracle.quant_rows_e4m3(oracle.decode_bf16(xb))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    qn = q.cpu().numpy()
    same = (qn == q_ref) | (((qn & 0x7F) == 0) & ((q_ref & 0x7F) == 0))     # +0 / -0
    assert same.all()


def test_activation_quantiser_rows_of_tiny_and_subnormal_values_stay_finite():
    """A row whose largest magnitude is tiny (below about 5.3e-36) would give a scale under 2^-126 and a reciprocal
    of +inf, turning the row's zeros into NaN bytes (0x7F) that poison the next GEMM: the scale is
    floored at 2^-126 instead (kernel and oracle alike)."""
    import cudaop_b200 as ops
    rows, cols = 6, 256
    x = np.zeros((rows, cols), np.float32)
    x[0, ::3] = 1e-37; x[0, 1::3] = -3e-38                     # below the threshold, zeros in between
    x[1, 5] = 9.2e-41                                          # the smallest bf16 subnormal alone
    x[2, :] = 1e-39; x[2, 7] = 0.0
    x[3, ::2] = 1e-35                                          # just above the threshold
    x[4, 3] = 1.0; x[4, 4] = 1e-40                             # an ordinary row with a subnormal element
    xb = oracle.encode_bf16(x)
    q, s = ops.quant_rows_e4m3(dev(xb, torch.bfloat16))
    torch.cuda.synchronize()
    qn, sn = q.cpu().numpy(), s.cpu().numpy()
    assert np.isfinite(sn).all() and (sn > 0).all()
    assert ((qn & 0x7F) != 0x7F).all()                         # no NaN byte anywhere
    q_ref, s_ref = oracle.quant_rows_e4m3(oracle.decode_bf16(xb))
    assert np.array_equal(sn.view(np.uint32), s_ref.view(np.uint32))
    assert ((qn == q_ref) | (((qn | q_ref) & 0x7F) == 0)).all()
    assert (qn[5] == 0).all() and sn[5] == 1.0                 # all-zero row: scale 1
