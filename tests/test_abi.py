"""CPU tests: the C-ABI library loads and exports every function its header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(rptc_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    from rptc_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert declared == set(_lib.exported_symbols()), "python binding table and header disagree"


def test_strerror_and_version_without_gpu():
    from rptc_b200 import lib
    assert lib().rptc_version() >= 100
    assert lib().rptc_strerror(0) == b"ok"
    assert b"aligned" in lib().rptc_strerror(-3)
    assert lib().rptc_strerror(-99) == b"unknown status"


def test_argument_errors_need_no_gpu():
    # argument validation happens before any CUDA call
    from rptc_b200 import Format, lib
    f = Format()
    assert lib().rptc_decompress(None, None, None, None, 0, 32, 64, ctypes.byref(f), None) == -1
    assert lib().rptc_gemv(1 << 8, 1 << 8, None, 1 << 8, 64, 1 << 8, 32, 31, 64, 1, 0, ctypes.byref(f), None) == -2
    assert lib().rptc_gemv(1 << 8, 1 << 8, None, 1 << 8, 64, 1 << 8, 32, 32, 64, 9, 0, ctypes.byref(f), None) == -1
    bad = Format(code=1, K=4)
    assert lib().rptc_decompress(1 << 8, 1 << 8, None, 1 << 8, 64, 32, 64, ctypes.byref(bad), None) == -4
    assert lib().rptc_hadamard(1 << 8, 0, 256, 1 << 8, 256, None, None, 0, 1, 256, 100, 0, 1.0, 0, None) == -1
    assert lib().rptc_repack(1 << 8, 0, 1 << 9, 2, 33, 4, None) == -2
