"""Builds cudaop_b200._C, the torch extension in front of libb200q.so, in place.

Layout follows the reference project's extensions (op/grouped_gemm/setup.py:18-46): a CUDAExtension named
``<package>._C`` built with ninja, -O3 / C++17.  The extension holds no kernels; it links the C-ABI library
``cudaop_b200/libb200q.so`` (built first by ``python -m cudaop_b200.build``) and finds it at run time next to
itself.  Use ``python -m cudaop_b200.build`` rather than calling this file directly: it builds the library,
sets TORCH_CUDA_ARCH_LIST=10.0a and checks that the module imports.
"""
from pathlib import Path

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "cudaop_b200"
SRC = PKG / "csrc_ext" / "ops.cpp"
if not SRC.is_file():
    raise FileNotFoundError(f"missing extension source: {SRC}")
if not (PKG / "libb200q.so").is_file():
    raise FileNotFoundError(f"{PKG / 'libb200q.so'} is missing: run `python -m cudaop_b200.build --lib` first")

setup(
    name="cudaop_b200",
    version="0.2.0",
    description="B200 (sm_100a) quantized GEMM operators behind CUDAOP's operator conventions",
    packages=["cudaop_b200"],
    ext_modules=[
        CUDAExtension(
            name="cudaop_b200._C",
            sources=[str(SRC.relative_to(ROOT))],
            include_dirs=[str(ROOT / "include")],
            library_dirs=[str(PKG)],
            libraries=["b200q"],
            extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": ["-O3", "-std=c++17"]},
            extra_link_args=["-Wl,-rpath,$ORIGIN"],
        ),
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
