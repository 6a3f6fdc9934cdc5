"""cudaop_b200 — Python entry points of the B200 quantized-GEMM library.

The package re-exports the torch extension ``cudaop_b200._C`` the way the reference project's
packages do (op/grouped_gemm/cudaop_grouped_gemm/__init__.py:3-24): tensor operators that take and
return ``torch.Tensor``s, validate device / dtype / contiguity / shape and raise on violation,
allocate the output on the input's device, and launch on torch's current stream
(op/grouped_gemm/csrc/grouped_gemm.cuh:106-176).  ``lib()`` gives ctypes access to the raw C ABI of
``libb200q.so`` (``include/b200q.h``) for callers that manage their own buffers, such as the
tensor-parallel MLP layer.  All arithmetic happens in ``libb200q.so`` (hand-written sm_100a CUDA);
there is no CPU or PyTorch fallback — a missing library or extension is an ImportError at first use.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")
_lib = None

__all__ = [
    "lib", "gemm_fp8", "gemm_i8", "gmm", "gmm_fp8", "GroupedFP8Weights", "gemm_fp8_rowcol", "gemm_fp8_swiglu", "gemm_w4a16", "gemm_nvfp4", "nvfp4_swizzle_sf",
    "gemm_mxfp8", "mxfp8_swizzle_sf", "quant_rows_nvfp4",
    "gemm_sparse_fp8", "quant_rows_e4m3", "status", "check_status", "set_wait_limit_ms", "WaitTimeout", "LIB_PATH",
]

_VP, _I, _F = C.c_void_p, C.c_int, C.c_float
_SIZE_T_FUNCS = {
    "b200q_gemm_nvfp4_workspace_bytes": [C.c_int, C.c_int, C.c_int],
    "b200q_nvfp4_sf_bytes": [C.c_int, C.c_int],
    "b200q_mxfp8_sf_bytes": [C.c_int, C.c_int],
    "b200q_gemm_mxfp8_workspace_bytes": [C.c_int, C.c_int, C.c_int],
    "b200q_gemm_nvfp4_static_max_bytes": [],
    "b200q_allreduce_signal_bytes": [],
    "b200q_rank_barrier_signal_bytes": [],
    "b200q_fused_allreduce_flag_bytes": [],
    "b200q_fused_allreduce_counter_bytes": [],
}
_SIGNATURES = {
    "b200q_gemm_fp8": [_VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_gemm_i8": [_VP, _VP, _VP, _VP, _I, _I, _I, _VP],
    "b200q_gmm_fp8": [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "b200q_gemm_fp8_rowcol": [_VP, _VP, _VP, _I, _I, _I, _VP, _VP, _I, _VP],
    "b200q_gemm_fp8_swiglu": [_VP, _VP, _VP, _VP, _I, _I, _I, _VP, _VP, _VP, _VP],
    "b200q_gemm_w4a16": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "b200q_gemm_nvfp4": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP, _VP],
    "b200q_gemm_nvfp4_static": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_gemm_nvfp4_blocked": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_nvfp4_swizzle_sf": [_VP, _VP, _I, _I, _VP],
    "b200q_gemm_mxfp8": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _VP, _VP],
    "b200q_gemm_mxfp8_blocked": [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _VP],
    "b200q_mxfp8_swizzle_sf": [_VP, _VP, _I, _I, _VP],
    "b200q_mxfp8_set_tile_n": [_I],
    "b200q_nvfp4_set_tile_n": [_I],
    "b200q_nvfp4_set_2cta": [_I],
    "b200q_fp8_set_tma_store": [_I],
    "b200q_fp8_set_dynamic_tiles": [_I],
    "b200q_fp8_set_group": [_I],
    "b200q_nvfp4_set_group": [_I],
    "b200q_sp24_set_2cta": [_I],
    "b200q_w4a16_set_impl": [_I],
    "b200q_w4a16_set_pdl": [_I],
    "b200q_sp24_set_tile_n": [_I],
    "b200q_gemm_sp24_fp8": [_VP, _VP, _VP, _VP, _I, _I, _I, _F, _F, _VP],
    "b200q_quant_rows_e4m3": [_VP, _VP, _VP, _I, _I, _VP],
    "b200q_quant_rows_nvfp4": [_VP, _VP, _VP, _I, _I, _F, _VP],
    "b200q_status": [_VP, _I],
    "b200q_set_wait_limit_ms": [_I, _I],
    "b200q_rank_barrier": [_VP, _I, _I, C.c_uint, C.c_uint, _VP],
    "b200q_reduce_scatter_to_bf16_one_device": [_VP, _VP, _VP, _I, C.c_longlong, C.c_longlong, _I, C.c_uint, C.c_uint, _I, _VP],
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
    "b200q_sum_to_bf16": [_VP, _I, _I, _VP, C.c_longlong, _I, _VP],
    "b200q_reduce_scatter_to_bf16": [_VP, _VP, _VP, _VP, _I, C.c_longlong, C.c_longlong, _I, _I, C.c_uint, C.c_uint, _I, _VP],
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


def _raise(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with cudaError {code}" + (" (invalid argument)" if code == 1 else ""))


def _check(t: torch.Tensor, name: str, dtypes, ndim: int) -> None:
    """Argument check for the few Python-level callers of the raw C ABI (the MLP layer)."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype not in dtypes or t.dim() != ndim or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CUDA tensor of {ndim} dimensions with dtype in {dtypes}")


# ---------------------------------------------------------------------------------------------------
# Tensor operators: the torch extension cudaop_b200._C (cudaop_b200/csrc_ext/ops.cpp, built by
# `python -m cudaop_b200.build`).  It validates its arguments (ValueError), guards the device, launches
# on torch's current stream and allocates the outputs; the functions below only give it Python
# signatures with defaults, as op/grouped_gemm/cudaop_grouped_gemm/ops.py does for its _C module.

EXTENSION_OPS = ("gemm_fp8", "gemm_fp8_rowcol", "gemm_fp8_swiglu", "gemm_w4a16", "nvfp4_swizzle_sf", "gemm_nvfp4",
                 "mxfp8_swizzle_sf", "gemm_mxfp8", "gemm_sparse_fp8", "quant_rows_e4m3", "quant_rows_nvfp4", "gemm_i8", "gmm_fp8")
try:
    from . import _C                                    # noqa: F401
    _C_ERROR = None
except ImportError as exc:                              # reported when an operator is first used
    _C, _C_ERROR = None, exc


def _ext():
    if _C is None:
        raise ImportError(f"the torch extension cudaop_b200._C is not built ({_C_ERROR}); run "
                          "`python -m cudaop_b200.build` (there is no fallback path)")
    return _C


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, scale_a: float, scale_b: float) -> torch.Tensor:
    """C[M,N] (bf16) = (A[M,K] @ B[N,K].T) * (scale_a * scale_b); A, B hold E4M3 bytes."""
    return _ext().gemm_fp8(a, b, float(scale_a), float(scale_b))


def gemm_i8(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None = None) -> torch.Tensor:
    """D[M,N] (int32) = A[M,K] (int8) @ B[N,K].T (int8) (+ C int32): exact integer GEMM on the tensor cores."""
    return _ext().gemm_i8(a, b, c)


def gmm_fp8(a_q, a_scale, b_q, b_scale, batch_sizes) -> torch.Tensor:
    """Grouped GEMM on quantised operands: a_q [tokens, K] E4M3 with per-token scales [tokens]; b_q [E, N, K] E4M3 with
    per-channel scales [E, N]; batch_sizes [E] int64 (CPU or CUDA): rows per group.  Returns [tokens, N] bf16; rows not
    covered by any group are zero."""
    return _ext().gmm_fp8(a_q, a_scale, b_q, b_scale, batch_sizes)


class GroupedFP8Weights:
    """Expert weights quantised once for :func:`gmm`: E4M3 bytes [E, N, K] (K contiguous) + fp32 scales [E, N],
    one per expert and output channel (max |w| / 448 over K)."""

    def __init__(self, b: torch.Tensor, trans_b: bool = False):
        if b.dim() != 3 or b.dtype != torch.bfloat16 or not b.is_cuda:
            raise ValueError("b must be a CUDA bf16 tensor [E, K, N] (trans_b=False) or [E, N, K] (trans_b=True)")
        w = b if trans_b else b.transpose(1, 2)
        w = w.contiguous()                                   # [E, N, K]
        E, N, K = w.shape
        q, s = quant_rows_e4m3(w.view(E * N, K))
        self.q, self.scale = q.view(E, N, K), s.view(E, N)
        self.E, self.N, self.K = E, N, K


def gmm(a: torch.Tensor, b, batch_sizes: torch.Tensor, trans_b: bool = False) -> torch.Tensor:
    """The reference's ``gmm(a, b, batch_sizes, trans_b)`` (op/grouped_gemm/cudaop_grouped_gemm/ops.py:76-83) on the
    FP8 tensor cores: ``a`` [tokens, K] bf16 is split into consecutive groups of ``batch_sizes[e]`` rows and group e
    is multiplied by expert e's weights.  ``b`` is a :class:`GroupedFP8Weights` (quantise once, reuse) or the
    reference's bf16 tensor — [E, K, N], or [E, N, K] with ``trans_b`` — which is then quantised on every call.
    Activations are quantised per token (E4M3), weights per output channel; the result is bf16 [tokens, N].
    Forward only (the reference's autograd wrapper has no quantised counterpart)."""
    w = b if isinstance(b, GroupedFP8Weights) else GroupedFP8Weights(b, trans_b)
    a_q, a_s = quant_rows_e4m3(a)
    return gmm_fp8(a_q, a_s, w.q, w.scale, batch_sizes)


def gemm_fp8_rowcol(a, b, row_scale, col_scale, out_dtype=torch.bfloat16) -> torch.Tensor:
    """C[m,n] = (A @ B.T)[m,n] * (row_scale[m] * col_scale[n]); bf16 or fp32 output."""
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be bfloat16 or float32")
    return _ext().gemm_fp8_rowcol(a, b, row_scale, col_scale, out_dtype == torch.float32)


def gemm_fp8_swiglu(x, w_gate, w_up, row_scale, gate_scale, up_scale) -> torch.Tensor:
    """H[M,I] (bf16) = silu(g) * u, g = (X @ Wg.T) * row_scale[m] * gate_scale[i], u likewise."""
    return _ext().gemm_fp8_swiglu(x, w_gate, w_up, row_scale, gate_scale, up_scale)


def gemm_w4a16(x, wq, scales, group: int = 128) -> torch.Tensor:
    """Y[M,N] (bf16) = X[M,K] (bf16) @ dequant(Wq[N,K/2], scales[N,K/group] fp16).T"""
    return _ext().gemm_w4a16(x, wq, scales, int(group))


def nvfp4_swizzle_sf(sf: torch.Tensor, K: int) -> torch.Tensor:
    """Row-major UE4M3 scales [rows, K/16] -> the blocked layout the GEMM reads (rewrite weights once)."""
    return _ext().nvfp4_swizzle_sf(sf, int(K))


def gemm_nvfp4(aq, sfa, bq, sfb, global_a: float, global_b: float, blocked: bool = False) -> torch.Tensor:
    """C[M,N] (bf16) for NVFP4 operands: packed E2M1 [rows,K/2], UE4M3 scales, fp32 global scales.

    Scales are row-major [rows, K/16] (``blocked=False``; a scratch buffer for their blocked copy is
    allocated per call) or the output of :func:`nvfp4_swizzle_sf` (``blocked=True``).
    """
    return _ext().gemm_nvfp4(aq, sfa, bq, sfb, float(global_a), float(global_b), bool(blocked))


def mxfp8_swizzle_sf(sf: torch.Tensor, K: int) -> torch.Tensor:
    """Row-major UE8M0 scales [rows, K/32] -> the blocked layout the MXFP8 GEMM reads."""
    return _ext().mxfp8_swizzle_sf(sf, int(K))


def gemm_mxfp8(a, sfa, b, sfb, blocked: bool = False) -> torch.Tensor:
    """C[M,N] (bf16) for MXFP8 operands: E4M3 bytes [rows, K] with one UE8M0 scale per 32 K ([rows, K/32], or the
    output of :func:`mxfp8_swizzle_sf` with ``blocked=True``)."""
    return _ext().gemm_mxfp8(a, sfa, b, sfb, bool(blocked))


def gemm_sparse_fp8(a_comp, a_meta, b, scale_a: float, scale_b: float) -> torch.Tensor:
    """C[M,N] (bf16) = (expand_2:4(a_comp[M,K/2], a_meta[M,K/8]) @ B[N,K].T) * (scale_a * scale_b)."""
    return _ext().gemm_sparse_fp8(a_comp, a_meta, b, float(scale_a), float(scale_b))


def quant_rows_e4m3(x: torch.Tensor):
    """bf16 [rows, cols] -> (E4M3 bytes [rows, cols] as uint8, fp32 scales [rows])."""
    return _ext().quant_rows_e4m3(x)


def quant_rows_nvfp4(x: torch.Tensor, global_scale: float):
    """bf16 [rows, cols] -> (packed E2M1 [rows, cols/2] uint8, UE4M3 scales in the blocked layout, 1-D uint8):
    operands for :func:`gemm_nvfp4` with ``blocked=True``."""
    return _ext().quant_rows_nvfp4(x, float(global_scale))


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
