"""Parity of the NVFP4 block-scaled GEMM (tcgen05 kind::mxf4nvf4) with the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[(128, 0), (192, 0), (256, 0), (192, 1), (256, 1)],
                ids=["one_cta_128", "one_cta_192", "one_cta_256", "cta_pair_192", "cta_pair_256"])
def tile_n(request):
    """Every kernel variant: one-CTA tiles of 128/192/256 columns and CTA-pair tiles (256 rows) of 192/256."""
    import cudaop_b200 as ops
    bn, pair = request.param
    ops.lib().b200q_nvfp4_set_tile_n(bn)
    ops.lib().b200q_nvfp4_set_2cta(pair)
    yield bn
    ops.lib().b200q_nvfp4_set_tile_n(256)
    ops.lib().b200q_nvfp4_set_2cta(1)


def _ref(aq, sfa, ga, bq, sfb, gb):
    return oracle.gemm_f32(oracle.dequant_nvfp4(aq, sfa, ga), oracle.dequant_nvfp4(bq, sfb, gb), threads=CORES)


def test_reference_known_answer_tile(tile_n):
    # op/test/arch_primitives/ptx_mma_fp4.cu:49-65,311-324: A nibbles 0x3 (+1.5), B nibbles 0x9 (-0.5),
    # scales {0.5,1,2,4} / {1,2,0.5,4}: sum over the four 16-blocks = -234 (the test's -233.75 minus its C of 0.25)
    import cudaop_b200 as ops
    M, N, K = 128, 256, 64
    aq = oracle.pack_u4(np.full((M, K), 0x3, np.uint8)); bq = oracle.pack_u4(np.full((N, K), 0x9, np.uint8))
    sfa = np.tile(np.array([0x30, 0x38, 0x40, 0x48], np.uint8), (M, 1))
    sfb = np.tile(np.array([0x38, 0x40, 0x30, 0x48], np.uint8), (N, 1))
    out = ops.gemm_nvfp4(dev(aq), dev(sfa), dev(bq), dev(sfb), 1.0, 1.0)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert np.all(bf16_to_f32(out) == -234.0)


def test_every_nibble_and_power_of_two_scales_exact(tile_n):
    # all 16 E2M1 codes and per-block power-of-two scales: every product and partial sum is exact
    # in fp32, so the only rounding is the final cast — the output must equal bf16(oracle) bit for bit
    import cudaop_b200 as ops
    M, N, K = 256, 448, 512
    rng = np.random.default_rng(0)
    aq = oracle.pack_u4(rng.integers(0, 16, (M, K), dtype=np.uint8))
    bq = oracle.pack_u4(rng.integers(0, 16, (N, K), dtype=np.uint8))
    sfa = (0x30 + 8 * rng.integers(0, 3, (M, K // 16))).astype(np.uint8)
    sfb = (0x30 + 8 * rng.integers(0, 3, (N, K // 16))).astype(np.uint8)
    out = ops.gemm_nvfp4(dev(aq), dev(sfa), dev(bq), dev(sfb), 1.0, 1.0)
    torch.cuda.synchronize()
    ref = oracle.gemm_f64acc(oracle.dequant_nvfp4(aq, sfa, 1.0), oracle.dequant_nvfp4(bq, sfb, 1.0), threads=CORES)
    assert np.array_equal(bf16_to_f32(out), oracle.decode_bf16(oracle.encode_bf16(ref.astype(np.float32))))


@pytest.mark.parametrize("shape", [(1, 8, 64), (128, 128, 64), (130, 200, 320), (260, 100, 128), (300, 520, 832),
                                   (512, 1024, 2048), (777, 1000, 1088)])
def test_quantised_normal_operands(tile_n, shape):
    import cudaop_b200 as ops
    M, N, K = shape
    aq, sfa, ga, bq, sfb, gb = oracle.make_nvfp4_case(M, N, K, seed=M + K)
    out = ops.gemm_nvfp4(dev(aq), dev(sfa), dev(bq), dev(sfb), ga, gb)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert_bar(bf16_to_f32(out), _ref(aq, sfa, ga, bq, sfb, gb), K, str(shape))


def test_scale_swizzle_is_the_documented_layout():
    import cudaop_b200 as ops
    rows, K = 200, 448
    sf = np.random.default_rng(1).integers(0, 127, (rows, K // 16), dtype=np.uint8)
    got = ops.nvfp4_swizzle_sf(dev(sf), K).cpu().numpy()
    k64 = K // 64
    want = np.zeros((2, k64, 512), np.uint8)
    for r in range(rows):
        for kb in range(k64):
            off = (r % 128 % 32) * 16 + (r % 128 // 32) * 4
            want[r // 128, kb, off:off + 4] = sf[r, 4 * kb:4 * kb + 4]
    assert np.array_equal(got, want.ravel())
    # blocked entry point gives the same result as the row-major one
    M, N = 200, 72
    aq, sfa, ga, bq, sfb, gb = oracle.make_nvfp4_case(M, N, K, seed=5)
    a = ops.gemm_nvfp4(dev(aq), dev(sfa), dev(bq), dev(sfb), ga, gb)
    b = ops.gemm_nvfp4(dev(aq), ops.nvfp4_swizzle_sf(dev(sfa), K), dev(bq), ops.nvfp4_swizzle_sf(dev(sfb), K), ga, gb,
                       blocked=True)
    assert torch.equal(a, b)


def test_config_8192_cubed_sampled_rows_and_global_scale_linearity():
    # M=N=K=8192, N(0,1) quantised to E2M1 with UE4M3 block scales and one fp32 global scale each
    import cudaop_b200 as ops
    S = 8192
    aq, sfa, ga, bq, sfb, gb = oracle.make_nvfp4_case(S, S, S, seed=0)
    a_d, b_d = dev(aq), dev(bq)
    sa_d, sb_d = ops.nvfp4_swizzle_sf(dev(sfa), S), ops.nvfp4_swizzle_sf(dev(sfb), S)
    out = ops.gemm_nvfp4(a_d, sa_d, b_d, sb_d, ga, gb, blocked=True)
    out4 = ops.gemm_nvfp4(a_d, sa_d, b_d, sb_d, 4.0 * ga, gb, blocked=True)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(out4.float(), out.float() * 4.0)
    rows = np.random.default_rng(0).choice(S, 256, replace=False)
    ref = oracle.gemm_f32(oracle.dequant_nvfp4(aq[rows], sfa[rows], ga), oracle.dequant_nvfp4(bq, sfb, gb), threads=CORES)
    rep = assert_bar(bf16_to_f32(out[torch.from_numpy(rows).cuda()]), ref, S, "nvfp4 8192^3 rows")
    print("nvfp4 8192^3", rep)


def test_argument_errors():
    import cudaop_b200 as ops
    L = ops.lib()
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    c = torch.zeros(128 * 128, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    p = z.data_ptr()
    assert L.b200q_gemm_nvfp4_blocked(p, p, p, p, c.data_ptr(), 16, 16, 48, 1.0, 1.0, st) == 1     # K % 64
    assert L.b200q_gemm_nvfp4_blocked(None, p, p, p, c.data_ptr(), 16, 16, 64, 1.0, 1.0, st) == 1
    assert L.b200q_gemm_nvfp4(p, p, p, p, c.data_ptr(), 16, 16, 64, 1.0, 1.0, None, st) == 1        # no workspace
    assert L.b200q_nvfp4_sf_bytes(129, 128) == 2 * 2 * 512 and L.b200q_nvfp4_sf_bytes(1, 60) == 0
    assert L.b200q_gemm_nvfp4_workspace_bytes(128, 256, 64) == 512 + 1024
    torch.cuda.synchronize()


@pytest.mark.parametrize("shape", [(1, 64), (130, 192), (300, 8192), (257, 3584), (64, 28672)])
def test_activation_quantiser_to_nvfp4_is_bit_exact(shape):
    """bf16 -> packed E2M1 + UE4M3 scales in the blocked layout, against the oracle's quantiser (same rule:
    sf = ue4m3((max/6)/g), q = e2m1(x * (1/(sf*g)))) and the library's own re-layout of the oracle's row-major scales."""
    import cudaop_b200 as ops
    rows, cols = shape
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * rng.uniform(0.05, 8.0, (rows, 1)).astype(np.float32)
    if rows > 2:
        x[2] = 0.0                                   # an all-zero row: zero scales, zero codes
        x[1, :16] = 0.0                              # an all-zero block inside a row
    xb = oracle.encode_bf16(x)
    xf = oracle.decode_bf16(xb)
    g = float(np.float32(np.abs(xf).max() / (6.0 * 448.0)))
    q, sf = ops.quant_rows_nvfp4(dev(xb, torch.bfloat16), g)
    torch.cuda.synchronize()
    q_ref, sf_ref = oracle.quant_nvfp4(xf, g)
    assert np.array_equal(sf.cpu().numpy(), ops.nvfp4_swizzle_sf(dev(sf_ref), cols).cpu().numpy())
    qn = q.cpu().numpy()
    lo, hi, lo_r, hi_r = qn & 0xF, qn >> 4, q_ref & 0xF, q_ref >> 4
    same = lambda a, b: (a == b) | (((a | b) & 7) == 0)          # +0 / -0
    assert same(lo, lo_r).all() and same(hi, hi_r).all()


def test_quantised_activations_feed_the_gemm():
    import cudaop_b200 as ops
    M, N, K = 200, 136, 512
    rng = np.random.default_rng(77)
    xa = oracle.encode_bf16(rng.standard_normal((M, K), dtype=np.float32))
    xw = oracle.encode_bf16(rng.standard_normal((N, K), dtype=np.float32))
    ga = float(np.float32(np.abs(oracle.decode_bf16(xa)).max() / (6.0 * 448.0)))
    gw = float(np.float32(np.abs(oracle.decode_bf16(xw)).max() / (6.0 * 448.0)))
    aq, sfa = ops.quant_rows_nvfp4(dev(xa, torch.bfloat16), ga)
    wq, sfw = ops.quant_rows_nvfp4(dev(xw, torch.bfloat16), gw)
    out = ops.gemm_nvfp4(aq, sfa, wq, sfw, ga, gw, blocked=True)
    torch.cuda.synchronize()
    aq_r, sfa_r = oracle.quant_nvfp4(oracle.decode_bf16(xa), ga)
    wq_r, sfw_r = oracle.quant_nvfp4(oracle.decode_bf16(xw), gw)
    ref = oracle.gemm_f32(oracle.dequant_nvfp4(aq_r, sfa_r, ga), oracle.dequant_nvfp4(wq_r, sfw_r, gw), threads=CORES)
    assert_bar(bf16_to_f32(out), ref, K, "quantise -> gemm")
    assert ops.status() == 0
