"""cudaop_b200._C, the torch extension: argument checks, device guard, current stream, results against the oracle.
Conventions checked are those of the reference's extensions (op/grouped_gemm/csrc/grouped_gemm.cuh:106-176)."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


def test_extension_module_is_the_in_tree_shared_object():
    import cudaop_b200 as ops
    assert ops._C is not None and "cudaop_b200" in ops._C.__file__ and ops._C.__file__.endswith(".so")


def test_operators_called_on_the_module_itself_match_the_oracle():
    import cudaop_b200 as ops
    C = ops._C
    # FP8, per-tensor scales
    aq, bq, sa, sb = oracle.make_fp8_case(136, 200, 256, seed=21)
    out = C.gemm_fp8(dev(aq), dev(bq).view(torch.float8_e4m3fn), sa, sb)      # uint8 or float8 views are both taken
    assert out.dtype == torch.bfloat16 and out.shape == (136, 200)
    ref = oracle.gemm_f32(oracle.decode_e4m3(aq) * np.float32(sa), oracle.decode_e4m3(bq) * np.float32(sb))
    assert_bar(bf16_to_f32(out), ref, 256, "_C.gemm_fp8")
    # W4A16
    xb, wq, s = oracle.make_w4a16_case(2, 64, 256, seed=22)
    y = C.gemm_w4a16(dev(xb, torch.bfloat16), dev(wq), dev(s, torch.float16), 128)
    assert_bar(bf16_to_f32(y), oracle.gemm_f32(oracle.decode_bf16(xb), oracle.dequant_w4(wq, s)), 256, "_C.gemm_w4a16")
    # NVFP4, row-major scales (workspace allocated inside) and blocked scales
    a4, sfa, ga, b4, sfb, gb = oracle.make_nvfp4_case(130, 72, 192, seed=23)
    ref = oracle.gemm_f32(oracle.dequant_nvfp4(a4, sfa, ga), oracle.dequant_nvfp4(b4, sfb, gb))
    c1 = C.gemm_nvfp4(dev(a4), dev(sfa), dev(b4), dev(sfb), ga, gb, False)
    c2 = C.gemm_nvfp4(dev(a4), C.nvfp4_swizzle_sf(dev(sfa), 192), dev(b4), C.nvfp4_swizzle_sf(dev(sfb), 192), ga, gb, True)
    assert torch.equal(c1, c2)
    assert_bar(bf16_to_f32(c1), ref, 192, "_C.gemm_nvfp4")
    # quantiser
    x = oracle.encode_bf16(np.random.default_rng(24).standard_normal((9, 64), dtype=np.float32))
    q, sc = C.quant_rows_e4m3(dev(x, torch.bfloat16))
    q_ref, s_ref = oracle.quant_rows_e4m3(oracle.decode_bf16(x))
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    qn = q.cpu().numpy()
    assert ((qn == q_ref) | (((qn | q_ref) & 0x7F) == 0)).all()
    torch.cuda.synchronize()
    assert ops.status() == 0


def test_argument_checks_raise_value_errors():
    import cudaop_b200 as ops
    a = torch.zeros((128, 128), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        ops.gemm_fp8(a.cpu(), a, 1.0, 1.0)                           # not a CUDA tensor
    with pytest.raises(ValueError):
        ops.gemm_fp8(a, a[:, :64], 1.0, 1.0)                         # inner dimensions differ
    with pytest.raises(ValueError):
        ops.gemm_fp8(a.t(), a, 1.0, 1.0)                             # not contiguous
    with pytest.raises(ValueError):
        ops.gemm_fp8(a.to(torch.int32), a, 1.0, 1.0)                 # dtype
    with pytest.raises(ValueError):
        ops.gemm_w4a16(torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda"), a, torch.zeros((128, 3), dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError):
        ops.quant_rows_e4m3(torch.zeros((4, 64), dtype=torch.float16, device="cuda"))
    torch.cuda.synchronize()


def test_a_refusal_by_the_c_abi_is_a_runtime_error():
    """An argument the tensor checks let through but the library refuses (here: a scale group size it does not
    implement) comes back as cudaErrorInvalidValue and must surface as an exception carrying that code."""
    import cudaop_b200 as ops
    x = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((32, 128), dtype=torch.uint8, device="cuda")
    s = torch.zeros((32, 4), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="cudaError 1"):
        ops.gemm_w4a16(x, w, s, 64)
    with pytest.raises(ValueError, match="inner dimensions differ: 128 vs 64"):
        a = torch.zeros((128, 128), dtype=torch.uint8, device="cuda")
        ops.gemm_fp8(a, a[:, :64].contiguous(), 1.0, 1.0)
    torch.cuda.synchronize()


def test_launches_on_the_current_stream():
    """The result of a call made on a side stream is complete once that stream is synchronised, with work queued
    in front of it on that stream only."""
    import cudaop_b200 as ops
    aq, bq, sa, sb = oracle.make_fp8_case(256, 256, 512, seed=25)
    a, b = dev(aq), dev(bq)
    want = ops.gemm_fp8(a, b, sa, sb)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    big = torch.empty((8192, 8192), device="cuda")
    with torch.cuda.stream(side):
        for _ in range(4):
            big.normal_()                                            # work in front of the GEMM on the side stream
        got = ops.gemm_fp8(a, b, sa, sb)
    side.synchronize()
    assert torch.equal(got, want)
    torch.cuda.synchronize()
