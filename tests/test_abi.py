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
    assert lib().rptc_gemv(1 << 8, 1 << 8, None, 1 << 8, 64, 1 << 8, 32, 32, 64, 65, 0, ctypes.byref(f), None) == -1    # 1..64 rows
    assert lib().rptc_gemv(1 << 8, 1 << 8, None, 1 << 8, 64, 1 << 8, 32, 32, 64, 0, 0, ctypes.byref(f), None) == -1
    bad = Format(code=1, K=4)
    assert lib().rptc_decompress(1 << 8, 1 << 8, None, 1 << 8, 64, 32, 64, ctypes.byref(bad), None) == -4
    assert lib().rptc_hadamard(1 << 8, 0, 256, 1 << 8, 256, None, None, 0, 1, 256, 100, 0, 1.0, 0, None) == -1
    assert lib().rptc_repack(1 << 8, 0, 1 << 9, 2, 33, 4, None) == -2


def test_entry_point_without_scratch_rejects_bad_calls_before_it_touches_its_array():
    """rptc_gemv_f16_static shares one array between all calls on a device: a call that is going to be refused must be
    refused before anything is queued on the caller's stream.  All of these return without a CUDA call."""
    from rptc_b200 import Format, lib
    f = Format()
    call = lib().rptc_gemv_f16_static
    ok = dict(codes=1 << 8, lut=1 << 8, x=1 << 8, ld_x=64, y=1 << 8, ld_y=32, m=32, n=64, batch=1, x_order=0, fmt=f)

    def status(**kw):
        a = {**ok, **kw}
        return call(a["codes"], a["lut"], None, a["x"], a["ld_x"], a["y"], a["ld_y"], a["m"], a["n"], a["batch"], a["x_order"],
                    ctypes.byref(a["fmt"]), None)

    assert status(codes=None) == -1                             # null codes
    assert status(y=None) == -1
    assert status(fmt=Format(code=7)) == -1                     # bad enum value
    assert status(fmt=Format(code=1, K=4)) == -4                # HASH is 2 bits per weight
    assert status(m=33) == -2                                   # m % 32
    assert status(codes=(1 << 8) + 4) == -3                     # codes not 16-byte aligned
    assert status(ld_x=32) == -2                                # ld_x < n
    assert status(m=262144 // 8 + 32, ld_y=1 << 20, batch=8) == -7      # beyond the fixed accumulator
    assert status(batch=9) == -1


def test_status_strings_cover_every_code():
    from rptc_b200 import lib
    for code in range(-10, 1):
        assert lib().rptc_strerror(code) != b"unknown status"
