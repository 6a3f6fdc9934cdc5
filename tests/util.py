"""Helpers shared by the GPU parity tests: host<->device moves and the acceptance bar."""
import os

import numpy as np
import torch

import oracle

CORES = os.cpu_count() or 1


def dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    elif a.dtype == np.uint32:
        a = a.view(np.int32)
    t = torch.from_numpy(a).cuda()
    return t if dtype is None else t.view(dtype)


def bf16_to_f32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()


def assert_bar(out_f32: np.ndarray, ref_f32: np.ndarray, k_dim: int, what: str = ""):
    """The bar: rel-Frobenius <= 1e-3 (against the oracle given the same final bf16 cast) and
    <= 2 bf16 ulp of the fp32 oracle (with the oracle's own summation-noise floor); see
    oracle.error_report for both definitions.  Returns the report."""
    rep = oracle.error_report(out_f32, ref_f32, k_dim=k_dim)
    assert rep["rel_fro"] <= 1e-3, (what, rep)
    assert rep["max_ulp_floor"] <= 2.0, (what, rep)
    return rep
