"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for f in os.listdir(os.path.join(ROOT, "include")):
        if f.endswith(".h"):
            src = open(os.path.join(ROOT, "include", f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names += re.findall(r"\b(?:int|void|size_t)\s+(b200q_\w+)\s*\(", src)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as g
    g.build()
    import cudaop_b200 as ops
    lib = ctypes.CDLL(ops.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 6
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"


def test_python_signatures_cover_the_header():
    import cudaop_b200 as ops
    for n in declared_symbols():
        assert n in ops._SIGNATURES or n in ops._SIZE_T_FUNCS, n


def test_missing_library_is_a_loud_error(monkeypatch):
    import cudaop_b200 as ops
    monkeypatch.setattr(ops, "_lib", None)
    monkeypatch.setattr(ops, "LIB_PATH", "/nonexistent/libb200q.so")
    try:
        ops.lib()
        assert False, "expected ImportError"
    except ImportError:
        pass


def test_torch_extension_is_built_in_tree_and_exports_every_operator():
    import __graft_entry__ as g
    g.build()
    import cudaop_b200 as ops
    assert ops._C is not None, ops._C_ERROR
    assert os.path.dirname(os.path.abspath(ops._C.__file__)) == os.path.join(ROOT, "cudaop_b200")
    for n in ops.EXTENSION_OPS:
        assert callable(getattr(ops._C, n)), n
        assert callable(getattr(ops, n)), n


def test_missing_extension_is_a_loud_error(monkeypatch):
    import cudaop_b200 as ops
    monkeypatch.setattr(ops, "_C", None)
    monkeypatch.setattr(ops, "_C_ERROR", ImportError("not built"))
    try:
        ops.gemm_fp8(None, None, 1.0, 1.0)
        assert False, "expected ImportError"
    except ImportError:
        pass


def test_extension_error_messages_with_numbers_are_exceptions_not_crashes():
    """Numbers in the extension's error messages are formatted with std::to_string: streaming them (the TORCH_CHECK
    default) crashed the process.  Checked here without a GPU through the dimension check, which comes first."""
    import pytest
    import torch
    import cudaop_b200 as ops
    with pytest.raises(ValueError, match="2 dimensions, got 1"):
        ops.gemm_fp8(torch.zeros(16, dtype=torch.uint8), torch.zeros((4, 16), dtype=torch.uint8), 1.0, 1.0)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.gemm_fp8(torch.zeros((4, 16), dtype=torch.uint8), torch.zeros((4, 16), dtype=torch.uint8), 1.0, 1.0)
