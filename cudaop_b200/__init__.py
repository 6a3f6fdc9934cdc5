"""cudaop_b200 — Python entry points of the B200 quantized-GEMM library.

The functions mirror the reference project's torch-extension conventions
(op/grouped_gemm/csrc/grouped_gemm.cuh:106-176, op/grouped_gemm/cudaop_grouped_gemm/__init__.py:3-24):
they take and return ``torch.Tensor``s, validate device / dtype / contiguity / shape and raise on
violation, allocate the output with the input's device, and launch on torch's current stream.
All arithmetic happens in ``libb200q.so`` (hand-written sm_100a CUDA behind a C ABI, see
``include/b200q.h``); there is no CPU or PyTorch fallback — a missing library is an ImportError at
first use.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")
_lib = None

__all__ = [
    "lib", "gemm_fp8", "gemm_fp8_rowcol", "gemm_fp8_swiglu", "gemm_w4a16", "gemm_nvfp4", "nvfp4_swizzle_sf",
    "gemm_sparse_fp8", "quant_rows_e4m3", "status", "check_status", "set_wait_limit_ms", "WaitTimeout", "LIB_PATH",
]

_VP, _I, _F = C.c_void_p, C.c_int, C.c_float
_SIZE_T_FUNCS = {
    "b200q_gemm_nvfp4_workspace_bytes": [C.c_int, C.c_int, C.c_int],
    "b200q_nvfp4_sf_bytes": [C.c_int, C.c_int],
    "b200q_gemm_nvfp4_static_max_bytes": [],
    "b200q_allreduce_signal_bytes": [],
    "b200q_fused_allreduce_flag_bytes": [],
    "b200q_fused_allreduce_counter_bytes": [],
}
_SIGNATURES = {
    "b200q_gemm_fp8": [_VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_gemm_fp8_rowcol": [_VP, _VP, _VP, _I, _I, _I, _VP, _VP, _I, _VP],
    "b200q_gemm_fp8_swiglu": [_VP, _VP, _VP, _VP, _I, _I, _I, _VP, _VP, _VP, _VP],
    "b200q_gemm_w4a16": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "b200q_gemm_nvfp4": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP, _VP],
    "b200q_gemm_nvfp4_static": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_gemm_nvfp4_blocked": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_nvfp4_swizzle_sf": [_VP, _VP, _I, _I, _VP],
    "b200q_nvfp4_set_tile_n": [_I],
    "b200q_nvfp4_set_2cta": [_I],
    "b200q_fp8_set_tma_store": [_I],
    "b200q_fp8_set_group": [_I],
    "b200q_nvfp4_set_group": [_I],
    "b200q_sp24_set_2cta": [_I],
    "b200q_w4a16_set_impl": [_I],
    "b200q_w4a16_set_pdl": [_I],
    "b200q_sp24_set_tile_n": [_I],
    "b200q_gemm_sp24_fp8": [_VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_quant_rows_e4m3": [_VP, _VP, _VP, _I, _I, _VP],
    "b200q_status": [_VP, _I],
    "b200q_set_wait_limit_ms": [_I, _I],
    "b200q_allreduce_to_bf16_one_device": [_VP, _VP, _VP, _I, C.c_longlong, C.c_longlong, _I, C.c_uint, C.c_uint, _I, _VP],
    "b200q_gemm_fp8_rowcol_allreduce_one_device": [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I,
                                                   C.c_uint, C.c_uint, _I, _I, _VP],
    "b200q_gemm_fp8_rowcol_allreduce": [_VP, _VP, _VP, _I, _I, _I, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _VP,
                                        C.c_uint, C.c_uint, _I, _I, _VP],
    "b200q_fp8_set_tile_n": [_I],
    "b200q_fp8_set_2cta": [_I],
    "b200q_fp8_set_sm_limit": [_I],
    "b200q_allreduce_set_reserved_smem": [_I],
    "b200q_fp8_set_reducer_stride": [_I],
    "b200q_allreduce_to_bf16": [_VP, _VP, _VP, _VP, _VP, _I, C.c_longlong, C.c_longlong, _I, _I, C.c_uint, C.c_uint, _I, _VP],
    "b200q_allreduce_set_unroll": [_I],
    "b200q_allreduce_set_threads": [_I],
}


def lib() -> C.CDLL:
    """Loads libb200q.so (built by ``python -m cudaop_b200.build``) and binds the C ABI."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m cudaop_b200.build` (there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        for name, args in _SIGNATURES.items():
            if hasattr(L, name):
                fn = getattr(L, name)
                fn.restype = _I
                fn.argtypes = args
        for name, args in _SIZE_T_FUNCS.items():
            if hasattr(L, name):
                fn = getattr(L, name)
                fn.restype = C.c_size_t
                fn.argtypes = args
        _lib = L
    return _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(t: torch.Tensor, name: str, dtypes, ndim: int) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dimensions, got {t.dim()}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _same_device(*ts: torch.Tensor) -> None:
    d = ts[0].device
    for t in ts[1:]:
        if t.device != d:
            raise ValueError("all tensors must be on the same device")


def _raise(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with cudaError {code}" + (" (invalid argument)" if code == 1 else ""))


_FP8 = (torch.uint8, torch.float8_e4m3fn)


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, scale_a: float, scale_b: float) -> torch.Tensor:
    """C[M,N] (bf16) = (A[M,K] @ B[N,K].T) * (scale_a * scale_b); A, B hold E4M3 bytes."""
    _check(a, "a", _FP8, 2); _check(b, "b", _FP8, 2); _same_device(a, b)
    M, K = a.shape; N, K2 = b.shape
    if K != K2:
        raise ValueError(f"inner dimensions differ: {K} vs {K2}")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        _raise(lib().b200q_gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                                    float(scale_a), float(scale_b), _stream()), "b200q_gemm_fp8")
    return out


def gemm_fp8_rowcol(a, b, row_scale, col_scale, out_dtype=torch.bfloat16) -> torch.Tensor:
    """C[m,n] = (A @ B.T)[m,n] * (row_scale[m] * col_scale[n]); bf16 or fp32 output."""
    _check(a, "a", _FP8, 2); _check(b, "b", _FP8, 2)
    _check(row_scale, "row_scale", (torch.float32,), 1); _check(col_scale, "col_scale", (torch.float32,), 1)
    _same_device(a, b, row_scale, col_scale)
    M, K = a.shape; N, K2 = b.shape
    if K != K2 or row_scale.numel() != M or col_scale.numel() != N:
        raise ValueError("shape mismatch")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be bfloat16 or float32")
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    with torch.cuda.device(a.device):
        _raise(lib().b200q_gemm_fp8_rowcol(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                                           row_scale.data_ptr(), col_scale.data_ptr(),
                                           int(out_dtype == torch.float32), _stream()), "b200q_gemm_fp8_rowcol")
    return out


def gemm_fp8_swiglu(x, w_gate, w_up, row_scale, gate_scale, up_scale) -> torch.Tensor:
    """H[M,I] (bf16) = silu(g) * u, g = (X @ Wg.T) * row_scale[m] * gate_scale[i], u likewise."""
    _check(x, "x", _FP8, 2); _check(w_gate, "w_gate", _FP8, 2); _check(w_up, "w_up", _FP8, 2)
    for n, t in (("row_scale", row_scale), ("gate_scale", gate_scale), ("up_scale", up_scale)):
        _check(t, n, (torch.float32,), 1)
    _same_device(x, w_gate, w_up, row_scale, gate_scale, up_scale)
    M, K = x.shape; I, K2 = w_gate.shape
    if K != K2 or tuple(w_up.shape) != (I, K) or row_scale.numel() != M or gate_scale.numel() != I or up_scale.numel() != I:
        raise ValueError("shape mismatch")
    out = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _raise(lib().b200q_gemm_fp8_swiglu(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(), M, I, K,
                                           row_scale.data_ptr(), gate_scale.data_ptr(), up_scale.data_ptr(),
                                           _stream()), "b200q_gemm_fp8_swiglu")
    return out


def gemm_w4a16(x, wq, scales, group: int = 128) -> torch.Tensor:
    """Y[M,N] (bf16) = X[M,K] (bf16) @ dequant(Wq[N,K/2], scales[N,K/group] fp16).T"""
    _check(x, "x", (torch.bfloat16,), 2); _check(wq, "wq", (torch.uint8,), 2); _check(scales, "scales", (torch.float16,), 2)
    _same_device(x, wq, scales)
    M, K = x.shape; N, K2 = wq.shape
    if K2 * 2 != K or K % group != 0 or tuple(scales.shape) != (N, K // group):
        raise ValueError("shape mismatch")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _raise(lib().b200q_gemm_w4a16(x.data_ptr(), wq.data_ptr(), scales.data_ptr(), out.data_ptr(), M, N, K,
                                      int(group), _stream()), "b200q_gemm_w4a16")
    return out


def nvfp4_swizzle_sf(sf: torch.Tensor, K: int) -> torch.Tensor:
    """Row-major UE4M3 scales [rows, K/16] -> the blocked layout the GEMM reads (rewrite weights once)."""
    _check(sf, "sf", (torch.uint8,), 2)
    rows = sf.shape[0]
    if sf.shape[1] * 16 != K or K % 64 != 0:
        raise ValueError("scales must be [rows, K/16] with K % 64 == 0")
    out = torch.empty((lib().b200q_nvfp4_sf_bytes(rows, K),), dtype=torch.uint8, device=sf.device)
    with torch.cuda.device(sf.device):
        _raise(lib().b200q_nvfp4_swizzle_sf(sf.data_ptr(), out.data_ptr(), rows, K, _stream()), "b200q_nvfp4_swizzle_sf")
    return out


def gemm_nvfp4(aq, sfa, bq, sfb, global_a: float, global_b: float, blocked: bool = False) -> torch.Tensor:
    """C[M,N] (bf16) for NVFP4 operands: packed E2M1 [rows,K/2], UE4M3 scales, fp32 global scales.

    Scales are row-major [rows, K/16] (``blocked=False``; a scratch buffer for their blocked copy is
    allocated per call) or the output of :func:`nvfp4_swizzle_sf` (``blocked=True``).
    """
    _check(aq, "aq", (torch.uint8,), 2); _check(bq, "bq", (torch.uint8,), 2)
    M, K2 = aq.shape; N, K2b = bq.shape; K = 2 * K2
    if K2 != K2b or K % 64 != 0:
        raise ValueError("shape mismatch (K must match and be a multiple of 64)")
    L = lib()
    out = torch.empty((M, N), dtype=torch.bfloat16, device=aq.device)
    if blocked:
        _check(sfa, "sfa", (torch.uint8,), 1); _check(sfb, "sfb", (torch.uint8,), 1)
        _same_device(aq, sfa, bq, sfb)
        if sfa.numel() != L.b200q_nvfp4_sf_bytes(M, K) or sfb.numel() != L.b200q_nvfp4_sf_bytes(N, K):
            raise ValueError("blocked scale arrays have the wrong size")
        with torch.cuda.device(aq.device):
            _raise(L.b200q_gemm_nvfp4_blocked(aq.data_ptr(), sfa.data_ptr(), bq.data_ptr(), sfb.data_ptr(),
                                              out.data_ptr(), M, N, K, float(global_a), float(global_b), _stream()),
                   "b200q_gemm_nvfp4_blocked")
        return out
    _check(sfa, "sfa", (torch.uint8,), 2); _check(sfb, "sfb", (torch.uint8,), 2)
    _same_device(aq, sfa, bq, sfb)
    if tuple(sfa.shape) != (M, K // 16) or tuple(sfb.shape) != (N, K // 16):
        raise ValueError("shape mismatch")
    ws = torch.empty((L.b200q_gemm_nvfp4_workspace_bytes(M, N, K),), dtype=torch.uint8, device=aq.device)
    with torch.cuda.device(aq.device):
        _raise(L.b200q_gemm_nvfp4(aq.data_ptr(), sfa.data_ptr(), bq.data_ptr(), sfb.data_ptr(), out.data_ptr(),
                                  M, N, K, float(global_a), float(global_b), ws.data_ptr(), _stream()),
               "b200q_gemm_nvfp4")
    return out


def gemm_sparse_fp8(a_comp, a_meta, b, scale_a: float, scale_b: float) -> torch.Tensor:
    """C[M,N] (bf16) = (expand_2:4(a_comp[M,K/2], a_meta[M,K/8]) @ B[N,K].T) * (scale_a * scale_b)."""
    _check(a_comp, "a_comp", _FP8, 2); _check(a_meta, "a_meta", (torch.uint8,), 2); _check(b, "b", _FP8, 2)
    _same_device(a_comp, a_meta, b)
    M, K2 = a_comp.shape; N, K = b.shape
    if K2 * 2 != K or tuple(a_meta.shape) != (M, K // 8):
        raise ValueError("shape mismatch")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=b.device)
    with torch.cuda.device(b.device):
        _raise(lib().b200q_gemm_sp24_fp8(a_comp.data_ptr(), a_meta.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                                         float(scale_a), float(scale_b), _stream()), "b200q_gemm_sp24_fp8")
    return out


def quant_rows_e4m3(x: torch.Tensor):
    """bf16 [rows, cols] -> (E4M3 bytes [rows, cols] as uint8, fp32 scales [rows])."""
    _check(x, "x", (torch.bfloat16,), 2)
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _raise(lib().b200q_quant_rows_e4m3(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, cols, _stream()),
               "b200q_quant_rows_e4m3")
    return q, s


def status(clear: bool = True) -> int:
    """Device status word: 0 unless a kernel gave up on a bounded wait (then its output is undefined)."""
    v = C.c_uint(0)
    _raise(lib().b200q_status(C.byref(v), int(clear)), "b200q_status")
    return v.value


def set_wait_limit_ms(ms: int, cross_rank: bool = False) -> None:
    """Limit of the kernels' bounded waits on the current device (inside the GPU, or on another rank's flags)."""
    _raise(lib().b200q_set_wait_limit_ms(int(cross_rank), int(ms)), "b200q_set_wait_limit_ms")


class WaitTimeout(RuntimeError):
    """A kernel gave up on a bounded wait; the outputs of that call are undefined."""


def check_status(what: str = "") -> None:
    """Synchronises the current device and raises WaitTimeout if any kernel gave up on a bounded wait."""
    w = status(clear=True)
    if w:
        site, cta = (w >> 24) & 0x7F, w & 0xFFFFFF
        raise WaitTimeout(f"{what + ': ' if what else ''}a kernel gave up waiting (site {site}, CTA {cta}); "
                          "its output is undefined")
