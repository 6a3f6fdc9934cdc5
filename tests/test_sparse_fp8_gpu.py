"""Parity of the 2:4 structured-sparse FP8 GEMM (tcgen05.mma.sp) with the CPU oracle, whose ground
truth is the dense product with the expanded A, as in the reference's sparse test."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[(128, 0), (192, 0), (256, 0), (192, 1)], ids=["one_cta_128", "one_cta_192", "one_cta_256", "cta_pair_224"])
def tile_n(request):
    """Every kernel variant: one-CTA tiles of 128/192/256 columns, and the CTA-pair kernel (256 x 224 tiles; problems of
    at most 128 rows still go to the one-CTA kernel)."""
    import cudaop_b200 as ops
    bn, pair = request.param
    ops.lib().b200q_sp24_set_tile_n(bn)
    ops.lib().b200q_sp24_set_2cta(pair)
    yield bn
    ops.lib().b200q_sp24_set_tile_n(192)
    ops.lib().b200q_sp24_set_2cta(1)


def _ref(comp, meta, bq, sa, sb):
    A = oracle.decode_e4m3(oracle.sp24_expand(comp, meta)) * np.float32(sa)
    return oracle.gemm_f32(A, oracle.decode_e4m3(bq) * np.float32(sb), threads=CORES)


def test_reference_known_answer_values(tile_n):
    # op/test/arch_primitives/ptx_mma_sparse.cu:128-147,163-184: every group keeps positions {0,1}
    # (metadata nibble 0x4), coordinate-dependent values, exact comparison with the dense product
    import cudaop_b200 as ops
    M, N, K = 128, 256, 256
    def ra(row, grp, idx):
        return float((row + grp) % 5 + 1) if idx == 0 else -float((row * 2 + grp) % 5 + 1)
    dense = np.zeros((M, K), np.float32)
    for r in range(M):
        for g in range(K // 4):
            dense[r, 4 * g] = ra(r, g, 0); dense[r, 4 * g + 1] = ra(r, g, 1)
    Bt = np.array([[float((k * 3 + c * 5 + 1) % 9 - 4) for k in range(K)] for c in range(N)], np.float32)
    comp, meta = oracle.sp24_compress(oracle.encode_e4m3(dense))
    assert np.all(meta == 0x44)
    out = ops.gemm_sparse_fp8(dev(comp), dev(meta), dev(oracle.encode_e4m3(Bt)), 1.0, 1.0)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert np.array_equal(bf16_to_f32(out), oracle.decode_bf16(oracle.encode_bf16(dense @ Bt.T)))


def test_all_six_position_pairs_exact(tile_n):
    import cudaop_b200 as ops
    M, N, K = 256, 448, 512
    rng = np.random.default_rng(0)
    pairs = np.array([[0, 1], [0, 2], [1, 2], [0, 3], [1, 3], [2, 3]])
    pick = pairs[rng.integers(0, 6, size=(M, K // 4))]
    mask = np.zeros((M, K // 4, 4), bool); np.put_along_axis(mask, pick, True, axis=2)
    A = np.where(mask.reshape(M, K), rng.integers(1, 4, (M, K)) * rng.choice([-1, 1], (M, K)), 0).astype(np.float32)
    B = rng.integers(-3, 4, (N, K)).astype(np.float32)
    comp, meta = oracle.sp24_compress(oracle.encode_e4m3(A))
    assert set(np.unique(meta & 0xF)) == {0x4, 0x8, 0x9, 0xC, 0xD, 0xE}
    out = ops.gemm_sparse_fp8(dev(comp), dev(meta), dev(oracle.encode_e4m3(B)), 1.0, 1.0)
    torch.cuda.synchronize()
    assert np.array_equal(bf16_to_f32(out), oracle.decode_bf16(oracle.encode_bf16(A @ B.T)))


@pytest.mark.parametrize("shape", [(1, 8, 128), (128, 192, 128), (130, 200, 384), (260, 100, 256), (300, 520, 896),
                                   (512, 1024, 2048), (4100, 260, 512)])
def test_quantised_normal_operands(tile_n, shape):
    import cudaop_b200 as ops
    M, N, K = shape
    comp, meta, bq, sa, sb = oracle.make_sparse_fp8_case(M, N, K, seed=M + K)
    out = ops.gemm_sparse_fp8(dev(comp), dev(meta), dev(bq), sa, sb)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert_bar(bf16_to_f32(out), _ref(comp, meta, bq, sa, sb), K, str(shape))


def test_sparse_equals_dense_kernel_on_expanded_operand():
    # the same product through the dense FP8 kernel on expand(A): identical accumulators
    import cudaop_b200 as ops
    M, N, K = 384, 512, 1024
    comp, meta, bq, sa, sb = oracle.make_sparse_fp8_case(M, N, K, seed=3)
    sp = ops.gemm_sparse_fp8(dev(comp), dev(meta), dev(bq), sa, sb)
    de = ops.gemm_fp8(dev(oracle.sp24_expand(comp, meta)), dev(bq), sa, sb)
    torch.cuda.synchronize()
    diff = (sp.float() - de.float()).abs().max().item()
    assert diff <= 2.0 ** -6 * de.float().abs().max().item()      # at most an ulp of bf16 from summation order


def test_config_4096_8192_8192_sampled_rows_and_linearity():
    import cudaop_b200 as ops
    M, N, K = 4096, 8192, 8192
    comp, meta, bq, sa, sb = oracle.make_sparse_fp8_case(M, N, K, seed=0)
    c_d, m_d, b_d = dev(comp), dev(meta), dev(bq)
    out = ops.gemm_sparse_fp8(c_d, m_d, b_d, sa, sb)
    out2 = ops.gemm_sparse_fp8(c_d, m_d, b_d, sa, 2.0 * sb)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(out2.float(), out.float() * 2.0)
    rows = np.random.default_rng(0).choice(M, 256, replace=False)
    rep = assert_bar(bf16_to_f32(out[torch.from_numpy(rows).cuda()]), _ref(comp[rows], meta[rows], bq, sa, sb), K,
                     "sparse rows")
    print("sparse fp8 4096x8192x8192", rep)


def test_argument_errors():
    import cudaop_b200 as ops
    L = ops.lib()
    z = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    c = torch.zeros(128 * 128, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    p = z.data_ptr()
    assert L.b200q_gemm_sp24_fp8(p, p, p, c.data_ptr(), 16, 16, 64, 1.0, 1.0, st) == 1      # K % 128
    assert L.b200q_gemm_sp24_fp8(p, None, p, c.data_ptr(), 16, 16, 128, 1.0, 1.0, st) == 1
    assert L.b200q_gemm_sp24_fp8(p, p, p, c.data_ptr(), 16, -1, 128, 1.0, 1.0, st) == 1
    torch.cuda.synchronize()
