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


def test_ctypes_mirrors_match_the_header_layout(tmp_path):
    """The Python side passes crl_config / crl_io / crl_linear_args by pointer: size and the offset of every field of
    the ctypes mirrors must be what a C compiler makes of the header (a field added on one side only would shift
    everything behind it without any error)."""
    import ctypes
    import shutil
    import subprocess
    import pytest
    from chessrl_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    mirrors = {"crl_config": _lib.Config, "crl_io": _lib.IO, "crl_linear_args": _lib.LinearArgs}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "chessrl_b200.h"', 'int main(void) {']
    for cname, cls in mirrors.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'  printf("{cname} {fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    want = {}
    for line in out.splitlines():
        cname, fname, value = line.split()
        want[(cname, fname)] = int(value)
    for cname, cls in mirrors.items():
        assert ctypes.sizeof(cls) == want[(cname, "size")], cname
        for fname, _ in cls._fields_:
            assert getattr(cls, fname).offset == want[(cname, fname)], (cname, fname)
