"""Parity of the MXFP8 block-scaled GEMM (E4M3 data, one UE8M0 scale per 32 K) with the oracle.
Format and known answer: op/test/arch_primitives/ptx_mma_fp8.cu:126-178 (all-ones E4M3 with scale 1.0 over K = 32
gives 32.0 everywhere), scale decoder op/test/arch_primitives/ptx_mma_fp6.cu:344-351."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


def _ref(aq, sfa, bq, sfb):
    return oracle.gemm_f32(oracle.dequant_mxfp8(aq, sfa), oracle.dequant_mxfp8(bq, sfb), threads=CORES)


def test_reference_known_answer_all_ones_tile_is_32():
    import cudaop_b200 as ops
    M, N, K = 16, 8, 32                                     # the reference's one-instruction tile
    a = np.full((M, K), 0x38, np.uint8); b = np.full((N, K), 0x38, np.uint8)
    sfa = np.full((M, 1), 127, np.uint8); sfb = np.full((N, 1), 127, np.uint8)
    out = ops.gemm_mxfp8(dev(a), dev(sfa), dev(b), dev(sfb))
    torch.cuda.synchronize()
    assert (out.float() == 32.0).all()
    # scales are powers of two applied per block: 2^3 on A and 2^-1 on B give 128
    out = ops.gemm_mxfp8(dev(a), dev(np.full((M, 1), 130, np.uint8)), dev(b), dev(np.full((N, 1), 126, np.uint8)))
    assert (out.float() == 128.0).all()
    assert ops.status() == 0


def test_every_scale_byte_position_is_used():
    """Each of the four 32-K steps of a 128-K slab takes its own scale byte: a value that differs per step and per
    row shows up exactly."""
    import cudaop_b200 as ops
    M, N, K = 130, 72, 256
    a = np.full((M, K), 0x38, np.uint8); b = np.full((N, K), 0x38, np.uint8)          # all ones
    sfa = (127 + (np.arange(M)[:, None] % 3) + np.arange(K // 32)[None, :] % 4).astype(np.uint8)
    sfb = (125 + (np.arange(N)[:, None] % 5) - np.arange(K // 32)[None, :] % 2).astype(np.uint8)
    out = ops.gemm_mxfp8(dev(a), dev(sfa), dev(b), dev(sfb)).float().cpu().numpy()
    want = 32.0 * (oracle.decode_ue8m0(sfa) @ oracle.decode_ue8m0(sfb).T)            # small powers of two: exact in bf16? no:
    want = oracle.decode_bf16(oracle.encode_bf16(want.astype(np.float32)))           # ... one RN-even cast, as the kernel's
    assert np.array_equal(out, want)


@pytest.mark.parametrize("shape", [(128, 128, 128), (300, 520, 832), (130, 72, 160), (1, 8, 32), (257, 200, 96),
                                   (1024, 1024, 1024)])
@pytest.mark.parametrize("bn", [256, 192])
def test_shapes_against_the_oracle(shape, bn):
    import cudaop_b200 as ops
    M, N, K = shape
    aq, sfa, bq, sfb = oracle.make_mxfp8_case(M, N, K, seed=M + N + K)
    assert ops.lib().b200q_mxfp8_set_tile_n(bn) == 0
    try:
        out = ops.gemm_mxfp8(dev(aq), dev(sfa), dev(bq), dev(sfb))
        sa, sb = ops.mxfp8_swizzle_sf(dev(sfa), K), ops.mxfp8_swizzle_sf(dev(sfb), K)
        out2 = ops.gemm_mxfp8(dev(aq), sa, dev(bq), sb, blocked=True)
        torch.cuda.synchronize()
    finally:
        ops.lib().b200q_mxfp8_set_tile_n(256)
    assert ops.status() == 0
    assert torch.equal(out, out2)
    assert_bar(bf16_to_f32(out), _ref(aq, sfa, bq, sfb), K, f"mxfp8 {shape} bn={bn}")


def test_full_size_sampled_rows_and_scale_linearity():
    import cudaop_b200 as ops
    S = 8192
    aq, sfa, bq, sfb = oracle.make_mxfp8_case(S, S, S, seed=7, spread=False)
    a, b = dev(aq), dev(bq)
    sa, sb = ops.mxfp8_swizzle_sf(dev(sfa), S), ops.mxfp8_swizzle_sf(dev(sfb), S)
    out = ops.gemm_mxfp8(a, sa, b, sb, blocked=True)
    torch.cuda.synchronize()
    assert ops.status() == 0
    rows = np.random.default_rng(3).choice(S, 256, replace=False)
    ref = oracle.gemm_f32(oracle.dequant_mxfp8(aq[rows], sfa[rows]), oracle.dequant_mxfp8(bq, sfb), threads=CORES)
    assert_bar(bf16_to_f32(out[torch.from_numpy(rows).cuda()]), ref, S, "mxfp8 8192^3 rows")
    # size-independent property over the whole matrix: raising every A scale by one doubles every output exactly
    sa2 = ops.mxfp8_swizzle_sf(dev((sfa + 1).astype(np.uint8)), S)
    out2 = ops.gemm_mxfp8(a, sa2, b, sb, blocked=True)
    torch.cuda.synchronize()
    assert torch.equal(out2.float(), out.float() * 2.0)


def test_argument_errors():
    import cudaop_b200 as ops
    a = torch.zeros((128, 96), dtype=torch.uint8, device="cuda")
    s = torch.zeros((128, 3), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        ops.gemm_mxfp8(a[:, :80].contiguous(), s, a[:, :80].contiguous(), s)       # K % 32
    with pytest.raises(ValueError):
        ops.gemm_mxfp8(a, s[:, :2].contiguous(), a, s)                               # scale shape
    torch.cuda.synchronize()
