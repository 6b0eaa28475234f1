"""The C-ABI library loads without a GPU and exports every function include/grws_b200.h declares."""
import ctypes
import os
import re

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "grws_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(grws_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_functions()
    for must in ("grws_spmm_fwd", "grws_csr_to_bcsr_count", "grws_bcsr_transpose_count", "grws_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from graph_rws_b200.core import _native
    lib = ctypes.CDLL(_native.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    # and the Python binding lists exactly the declared functions
    assert sorted(_native.SIGNATURES) == declared_functions()


def test_argument_errors_are_reported_without_a_gpu():
    from graph_rws_b200.core import _native
    lib = _native.lib()
    assert lib.grws_version() >= 100
    # N not a multiple of 8 is rejected before any CUDA call
    st = lib.grws_spmm_fwd(16, 16, 16, 0, 16, 0, 8, 16, 0, 8, 1, 1, 4, 7, 16, 0, 0, None)
    assert st == -1 and b"multiple of 8" in lib.grws_last_error()
    st = lib.grws_spmm_fwd(16, 16, 16, 1, 16, 2, 8, 16, 0, 8, 1, 1, 4, 8, 16, 0, 0, None)
    assert st == -2
