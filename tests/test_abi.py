"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import os
import re

from conftest import ROOT


def test_exports_match_header(lib):
    header = open(os.path.join(ROOT, "include", "chessrl_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = sorted(set(re.findall(r"\b(crl_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    from chessrl_b200 import _lib
    assert sorted(_lib.EXPORTS) == declared


def test_argument_errors_without_gpu(lib):
    import ctypes
    assert lib.crl_strerror(0) == b"ok" and lib.crl_strerror(-4) == b"missing weight"
    assert lib.crl_create(None, 0, None) == -1
    assert lib.crl_num_moves(None) == 0 and lib.crl_workspace_bytes(None, 8) == 0
    st = ctypes.c_int(0)
    assert lib.crl_last_status(None, ctypes.byref(st)) == -1
    assert lib.crl_linear(7, None, 0, None, 0, None, 0, 0, 1, 1, 1, None, None, 0, 1.0, 0, None, None) == -1
