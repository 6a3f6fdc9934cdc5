"""Generates tests/golden/gemm_mma_cpu.npz by running the reference's own compiled
CPU GEMM (oracle/_ref/libcudaop_ref.so, built by `make -C oracle ref` from the
reference's op/cpu/cpu_ops.cpp) on small seeded inputs.  Run in a container that has
the reference tree mounted:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle  # noqa: E402

oracle.build(force=True)
assert oracle.ref_lib() is not None, "reference tree not mounted"
rng = np.random.default_rng(20260720)
out = {}
for i, (M, N, K) in enumerate([(1, 1, 1), (3, 5, 7), (16, 8, 32), (17, 23, 301), (32, 48, 1024)]):
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    out[f"A{i}"] = A; out[f"B{i}"] = B
    out[f"C{i}"] = oracle.gemm_f32(A, B, use_reference=True)
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemm_mma_cpu.npz"), **out)
print("wrote gemm_mma_cpu.npz", {k: v.shape for k, v in out.items() if k.startswith("C")})
