"""Parity of the FP8 E4M3 GEMM (tcgen05 kernel behind the C ABI) with the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[(1, 1), (1, 0), (0, 0)], ids=["cta_pair", "cta_pair_direct_stores", "one_cta"], autouse=True)
def kernel_variant(request):
    """The FP8 kernels: CTA pairs (tcgen05 cta_group::2, default; results through TMA stores or stored
    straight from registers) and the one-CTA kernel."""
    import cudaop_b200 as ops
    pair, tma_store = request.param
    ops.lib().b200q_fp8_set_2cta(pair)
    ops.lib().b200q_fp8_set_tma_store(tma_store)
    yield request.param
    ops.lib().b200q_fp8_set_2cta(1)
    ops.lib().b200q_fp8_set_tma_store(1)


def _run(aq, bq, sa, sb):
    import cudaop_b200 as ops
    out = ops.gemm_fp8(dev(aq), dev(bq), sa, sb)
    torch.cuda.synchronize()
    assert ops.status() == 0
    return bf16_to_f32(out)


def _oracle(aq, bq, sa, sb):
    A = oracle.decode_e4m3(aq) * np.float32(sa)
    B = oracle.decode_e4m3(bq) * np.float32(sb)
    return oracle.gemm_f32(A, B, threads=CORES)


def test_all_ones_tile_known_answer():
    # op/test/arch_primitives/ptx_mma_fp8.cu:48-59: ones (0x38) contract to K exactly
    for (M, N, K) in [(16, 8, 32), (128, 256, 128), (128, 256, 512)]:
        out = _run(np.full((M, K), 0x38, np.uint8), np.full((N, K), 0x38, np.uint8), 1.0, 1.0)
        assert np.all(out == float(K)), (M, N, K, out[:2, :4])


def test_coordinate_dependent_integers_exact():
    # small integers, exactly representable in E4M3, fp32 and (the results) bf16: any error in
    # the swizzle, descriptor stepping or TMEM lane/column map shows as a wrong integer
    M, N, K = 256, 512, 256
    A = np.array([[((r * 3 + k * 5 + 1) % 5) - 2 for k in range(K)] for r in range(M)], np.float32)
    B = np.array([[((n * 7 + k * 2 + 3) % 3) - 1 for k in range(K)] for n in range(N)], np.float32)
    out = _run(oracle.encode_e4m3(A), oracle.encode_e4m3(B), 1.0, 1.0)
    want = oracle.gemm_f32(A, B, threads=CORES)
    assert np.abs(want).max() <= 256          # exact in bf16
    assert np.array_equal(out, want)


def test_config_1024_cubed_against_oracle():
    # M=N=K=1024, N(0,1) scaled to +-448 with one fp32 per-tensor scale each, seed 0
    aq, bq, sa, sb = oracle.make_fp8_case(1024, 1024, 1024, seed=0)
    rep = assert_bar(_run(aq, bq, sa, sb), _oracle(aq, bq, sa, sb), 1024, "fp8 1024^3")
    print("fp8 1024^3", rep)


@pytest.mark.parametrize("shape", [(1, 8, 16), (5, 3, 16), (127, 255, 112), (129, 257, 144),
                                   (300, 520, 1040), (128, 256, 4096), (2048, 1024, 128)])
def test_ragged_and_edge_shapes(shape):
    M, N, K = shape
    aq, bq, sa, sb = oracle.make_fp8_case(M, N, K, seed=M + N + K)
    assert_bar(_run(aq, bq, sa, sb), _oracle(aq, bq, sa, sb), K, str(shape))


def test_output_is_not_written_outside_the_matrix():
    import cudaop_b200 as ops
    M, N, K = 130, 264, 128
    aq, bq, sa, sb = oracle.make_fp8_case(M, N, K, seed=9)
    buf = torch.full((M + 2, N), -7.0, dtype=torch.bfloat16, device="cuda")
    a_d, b_d = dev(aq), dev(bq)
    code = ops.lib().b200q_gemm_fp8(a_d.data_ptr(), b_d.data_ptr(), buf[1:].data_ptr(), M, N, K,
                                    sa, sb, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == 0
    assert torch.all(buf[0] == -7.0) and torch.all(buf[M + 1] == -7.0)
    assert_bar(bf16_to_f32(buf[1:M + 1]), _oracle(aq, bq, sa, sb), K)


def test_full_size_8192_sampled_rows_and_linearity():
    # full benchmark size: 256 seeded rows against the oracle, the whole matrix through a
    # size-independent property (doubling one scale doubles every output exactly)
    import cudaop_b200 as ops
    M = N = K = 8192
    aq, bq, sa, sb = oracle.make_fp8_case(M, N, K, seed=0)
    a_d, b_d = dev(aq), dev(bq)
    out = ops.gemm_fp8(a_d, b_d, sa, sb)
    out2 = ops.gemm_fp8(a_d, b_d, 2.0 * sa, sb)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(out2.float(), out.float() * 2.0)
    rows = np.random.default_rng(0).choice(M, 256, replace=False)
    A = oracle.decode_e4m3(aq[rows]) * np.float32(sa)
    B = oracle.decode_e4m3(bq) * np.float32(sb)
    rep = assert_bar(bf16_to_f32(out[torch.from_numpy(rows).cuda()]), oracle.gemm_f32(A, B, threads=CORES), K,
                     "fp8 8192^3 rows")
    print("fp8 8192^3", rep)
    # every row: compare with an fp32 GEMM of the same dequantised operands on the device
    ref = (torch.from_numpy(oracle.decode_e4m3(aq)).cuda() * sa) @ (torch.from_numpy(oracle.decode_e4m3(bq)).cuda() * sb).T
    err = (out.float() - ref.to(torch.bfloat16).float()).norm() / ref.norm()   # same final cast on both sides
    assert err.item() <= 1e-3, err.item()


def test_rowcol_scales_and_fp32_output():
    import cudaop_b200 as ops
    M, N, K = 200, 300, 512
    rng = np.random.default_rng(3)
    aq = oracle.encode_e4m3(rng.standard_normal((M, K), dtype=np.float32))
    bq = oracle.encode_e4m3(rng.standard_normal((N, K), dtype=np.float32))
    rs = rng.uniform(0.5, 2.0, M).astype(np.float32); cs = rng.uniform(0.001, 0.01, N).astype(np.float32)
    ref = oracle.gemm_f32(oracle.decode_e4m3(aq), oracle.decode_e4m3(bq), threads=CORES) * (rs[:, None] * cs[None, :])
    o16 = ops.gemm_fp8_rowcol(dev(aq), dev(bq), dev(rs), dev(cs))
    o32 = ops.gemm_fp8_rowcol(dev(aq), dev(bq), dev(rs), dev(cs), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert_bar(bf16_to_f32(o16), ref, K)
    np.testing.assert_allclose(o32.cpu().numpy(), ref, rtol=2e-5, atol=1e-6 * np.abs(ref).max())
    assert torch.equal(o32.to(torch.bfloat16), o16)


def test_swiglu_epilogue():
    import cudaop_b200 as ops
    M, I, K = 150, 384, 256
    rng = np.random.default_rng(4)
    xq = oracle.encode_e4m3(rng.standard_normal((M, K), dtype=np.float32))
    wg = oracle.encode_e4m3(rng.standard_normal((I, K), dtype=np.float32))
    wu = oracle.encode_e4m3(rng.standard_normal((I, K), dtype=np.float32))
    rs = rng.uniform(0.005, 0.02, M).astype(np.float32)
    sg = rng.uniform(0.5, 2.0, I).astype(np.float32); su = rng.uniform(0.5, 2.0, I).astype(np.float32)
    X = oracle.decode_e4m3(xq)
    g = oracle.gemm_f32(X, oracle.decode_e4m3(wg), threads=CORES) * (rs[:, None] * sg[None, :])
    u = oracle.gemm_f32(X, oracle.decode_e4m3(wu), threads=CORES) * (rs[:, None] * su[None, :])
    ref = oracle.swiglu(g, u)
    out = ops.gemm_fp8_swiglu(dev(xq), dev(wg), dev(wu), dev(rs), dev(sg), dev(su))
    torch.cuda.synchronize()
    assert ops.status() == 0
    rep = oracle.error_report(bf16_to_f32(out), ref, k_dim=K)
    assert rep["rel_fro"] <= 1e-3 and rep["max_ulp_floor"] <= 2.0, rep


def test_argument_errors_follow_the_reference_convention():
    # op/topk/topk_cuda.cu:239-246: null pointers and non-positive sizes -> cudaErrorInvalidValue
    import cudaop_b200 as ops
    L = ops.lib()
    a = torch.zeros(128, 128, dtype=torch.uint8, device="cuda")
    c = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert L.b200q_gemm_fp8(None, a.data_ptr(), c.data_ptr(), 128, 128, 128, 1.0, 1.0, s) == 1
    assert L.b200q_gemm_fp8(a.data_ptr(), a.data_ptr(), c.data_ptr(), 0, 128, 128, 1.0, 1.0, s) == 1
    assert L.b200q_gemm_fp8(a.data_ptr(), a.data_ptr(), c.data_ptr(), 128, 128, 24, 1.0, 1.0, s) == 1   # K % 16
    assert L.b200q_gemm_fp8(a.data_ptr() + 1, a.data_ptr(), c.data_ptr(), 64, 64, 64, 1.0, 1.0, s) == 1  # alignment
    with pytest.raises(ValueError):
        ops.gemm_fp8(a.cpu(), a, 1.0, 1.0)
    with pytest.raises(ValueError):
        ops.gemm_fp8(a, a[:, :64], 1.0, 1.0)
    torch.cuda.synchronize()
