"""ctypes front end of the C oracle (oracle/rptc_oracle.c).  TEST / BASELINE INFRASTRUCTURE ONLY.

Builds oracle/_build/librptc_oracle.so with `make -C oracle` on first use when it is missing.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "librptc_oracle.so")
_lib = None


def build() -> str:
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        L.rptc_oracle_threads.restype = ctypes.c_int
        p, i64, i = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        L.rptc_oracle_decompress.argtypes = [p, i, p, p, p, i64, i64, i, i, i, i]
        L.rptc_oracle_decompress.restype = i
        L.rptc_oracle_gemv.argtypes = [p, i, p, p, p, p, p, i64, i64, i, i, i, i, i]
        L.rptc_oracle_gemv.restype = i
        _lib = L
    return _lib


def threads() -> int:
    return lib().rptc_oracle_threads()


def set_threads(n: int) -> None:
    lib().rptc_oracle_set_threads(int(n))


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def decompress(codes: np.ndarray, lut: np.ndarray, m: int, n: int, code: int = 0, K: int = 2, L: int = 16,
               S: int = 8, layout: int = 0, carry_in: np.ndarray | None = None) -> np.ndarray:
    codes = np.ascontiguousarray(codes).view(np.uint32)
    lut = np.ascontiguousarray(lut, dtype=np.float16)
    ci = None if carry_in is None else np.ascontiguousarray(carry_in, dtype=np.uint32)
    out = np.empty((m, n), dtype=np.float16)
    rc = lib().rptc_oracle_decompress(_ptr(codes), layout, _ptr(lut), _ptr(ci), _ptr(out), m, n, code, K, L, S)
    assert rc == 0
    return out


def gemv(codes: np.ndarray, lut: np.ndarray, x: np.ndarray, m: int, n: int, code: int = 0, K: int = 2,
         L: int = 16, S: int = 8, layout: int = 0, carry_in: np.ndarray | None = None) -> np.ndarray:
    codes = np.ascontiguousarray(codes).view(np.uint32)
    lut = np.ascontiguousarray(lut, dtype=np.float16)
    x = np.ascontiguousarray(x, dtype=np.float16).reshape(-1, n)
    ci = None if carry_in is None else np.ascontiguousarray(carry_in, dtype=np.uint32)
    y = np.empty((x.shape[0], m), dtype=np.float32)
    scratch = np.empty(threads() * n, dtype=np.uint16)
    rc = lib().rptc_oracle_gemv(_ptr(codes), layout, _ptr(lut), _ptr(ci), _ptr(x), _ptr(y), _ptr(scratch),
                                m, n, x.shape[0], code, K, L, S)
    assert rc == 0
    return y
