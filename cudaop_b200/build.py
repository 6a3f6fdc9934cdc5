"""Builds libb200q.so (the C-ABI library) and the per-operator benchmark executables
in-tree with nvcc for sm_100a.  No GPU is needed to build.

    python -m cudaop_b200.build            # library + torch extension + executables
    python -m cudaop_b200.build --lib      # library only

The torch extension cudaop_b200._C is built by the repository's setup.py (CUDAExtension, ninja) with
TORCH_CUDA_ARCH_LIST=10.0a and import-checked afterwards, as the reference's build scripts do
(op/grouped_gemm/build.py:15-53, op/lora_moe/build.py:53-67).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
BENCH = os.path.join(HERE, "bench")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libb200q.so")

NVCC = os.environ.get("NVCC", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ARCH + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
                 "-I", os.path.join(ROOT, "include")]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd: list[str], log: str | None = None) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("command failed: " + " ".join(cmd))


def build_lib(force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "b200q.h"))
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJ, s[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [os.path.join(CSRC, s)] + headers):
            jobs.append(([NVCC] + CFLAGS + ["-c", os.path.join(CSRC, s), "-o", o], o[:-2] + ".ptxas.log"))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda j: _run(*j), jobs))
    if jobs or not os.path.exists(LIB):
        _run([NVCC] + ARCH + ["-shared", "-o", LIB] + objs)
    return LIB


def build_bench(force: bool = False) -> list[str]:
    outs = []
    if not os.path.isdir(BENCH):
        return outs
    for s in sorted(f for f in os.listdir(BENCH) if f.endswith(".cu")):
        exe = os.path.join(BENCH, s[:-3])
        deps = [os.path.join(BENCH, s), LIB] + [os.path.join(BENCH, h) for h in os.listdir(BENCH) if h.endswith(".h")]
        if force or _newer(exe, deps):
            extra = ["-lnccl"] if "nccl" in s else []
            _run([NVCC] + CFLAGS + [os.path.join(BENCH, s), "-o", exe, "-L", HERE, "-lb200q",
                                    "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."] + extra)
        outs.append(exe)
    return outs


def build_ext(force: bool = False) -> str:
    """cudaop_b200/_C*.so via setup.py build_ext --inplace; then checks that the module imports and exports
    every operator."""
    import glob
    src = os.path.join(HERE, "csrc_ext", "ops.cpp")
    deps = [src, LIB, os.path.join(ROOT, "include", "b200q.h"), os.path.join(ROOT, "setup.py")]
    found = glob.glob(os.path.join(HERE, "_C*.so"))
    if force or not found or _newer(found[0], deps):
        env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0a", MAX_JOBS=os.environ.get("MAX_JOBS", "8"))
        r = subprocess.run([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=ROOT, env=env,
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout)
            raise RuntimeError("building cudaop_b200._C failed")
        found = glob.glob(os.path.join(HERE, "_C*.so"))
    # import check in a fresh interpreter (this process may hold an older copy of the module)
    code = ("import sys; sys.path.insert(0, %r); import cudaop_b200 as ops; "
            "missing = [n for n in ops.EXTENSION_OPS if not callable(getattr(ops._C, n, None))]; "
            "assert ops._C is not None, ops._C_ERROR; assert not missing, missing" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("cudaop_b200._C does not import or lacks operators")
    return found[0]


def main() -> None:
    force = "--force" in sys.argv
    print(build_lib(force))
    if "--lib" not in sys.argv:
        print(build_ext(force))
        for e in build_bench(force):
            print(e)


if __name__ == "__main__":
    main()
