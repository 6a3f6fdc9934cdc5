"""b200q_gemm_nvfp4_static — the NVFP4 GEMM for callers that cannot allocate device memory.

A plug-in inside a server that owns the whole GPU's memory pool, or a loop that must never touch
the CUDA allocator, cannot supply the scratch buffer the regular entry point asks for; the static
entry point keeps that scratch in an array inside the library.  This file is collected last on
purpose, and it must pass both on its own in a fresh process and after every other test.
"""
import numpy as np
import pytest
import torch

import oracle
from tests.util import dev

pytestmark = pytest.mark.gpu


def _both(case, M, N, K):
    """Runs the regular (caller-owned workspace) and the static entry point on the same operands."""
    import cudaop_b200 as ops
    L = ops.lib()
    aq, sfa, ga, bq, sfb, gb = case
    a, sa, b, sb = dev(aq), dev(sfa), dev(bq), dev(sfb)
    st = torch.cuda.current_stream().cuda_stream
    ws = torch.empty((L.b200q_gemm_nvfp4_workspace_bytes(M, N, K),), dtype=torch.uint8, device="cuda")
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert L.b200q_gemm_nvfp4(a.data_ptr(), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), want.data_ptr(), M, N, K,
                              ga, gb, ws.data_ptr(), st) == 0
    assert L.b200q_gemm_nvfp4_static(a.data_ptr(), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), got.data_ptr(), M, N, K,
                                     ga, gb, st) == 0
    torch.cuda.synchronize()
    assert ops.status() == 0
    return got, want


def test_static_entry_matches_the_workspace_entry_on_two_calls_in_a_row():
    # first call: ragged row blocks, fills a large part of the built-in array
    M, N, K = 300, 520, 832
    got, want = _both(oracle.make_nvfp4_case(M, N, K, seed=41), M, N, K)
    assert torch.equal(got, want)           # same kernels on the same bytes: identical, not merely close
    # second call straight after it: a smaller problem over the array's stale contents
    M, N, K = 130, 72, 192
    got, want = _both(oracle.make_nvfp4_case(M, N, K, seed=42), M, N, K)
    assert torch.equal(got, want)
    # and the result is right, not just self-consistent
    aq, sfa, ga, bq, sfb, gb = oracle.make_nvfp4_case(M, N, K, seed=42)
    ref = oracle.gemm_f32(oracle.dequant_nvfp4(aq, sfa, ga), oracle.dequant_nvfp4(bq, sfb, gb))
    rep = oracle.error_report(got.float().cpu().numpy(), ref, k_dim=K)
    assert rep["rel_fro"] <= 1e-3 and rep["max_ulp_floor"] <= 2.0, rep


def test_static_entry_takes_no_device_memory_once_warm():
    """After one warm-up call (which loads the kernels' images and looks up the array's address) further
    calls leave the driver's count of free device memory exactly where it was."""
    import cudaop_b200 as ops
    L = ops.lib()
    M, N, K = 256, 384, 512
    aq, sfa, ga, bq, sfb, gb = oracle.make_nvfp4_case(M, N, K, seed=43)
    a, sa, b, sb = dev(aq), dev(sfa), dev(bq), dev(sfb)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def call():
        assert L.b200q_gemm_nvfp4_static(a.data_ptr(), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), out.data_ptr(),
                                         M, N, K, ga, gb, st) == 0
    call()                                      # warm-up: module load, function attributes, symbol address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert ops.status() == 0


def test_static_entry_refuses_problems_beyond_its_array():
    import cudaop_b200 as ops
    L = ops.lib()
    limit = L.b200q_gemm_nvfp4_static_max_bytes()
    assert limit == 8 << 20
    assert L.b200q_gemm_nvfp4_workspace_bytes(8192, 8192, 8192) == limit          # the largest square that fits
    z = torch.zeros(64, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    p = z.data_ptr()
    # one more row block than fits: refused before anything is launched (cudaErrorInvalidValue = 1)
    assert L.b200q_gemm_nvfp4_static(p, p, p, p, p, 8192 + 128, 8192, 8192, 1.0, 1.0, st) == 1
    assert L.b200q_gemm_nvfp4_static(p, p, p, p, p, 128, 128, 100, 1.0, 1.0, st) == 1    # K % 64
    torch.cuda.synchronize()
