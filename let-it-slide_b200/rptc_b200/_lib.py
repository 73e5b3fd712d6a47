"""ctypes binding of librptc_b200.so (include/rptc_b200.h).

The library is the product: there is no CPU or PyTorch fallback.  Importing this module without
the built library, or calling it on a machine without a compute-capability-10 GPU, raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("RPTC_B200_LIB") or os.path.join(_PKG, "librptc_b200.so")

CODE_LUT, CODE_HASH, CODE_LITE = 0, 1, 2
LAYOUT_ROWMAJOR, LAYOUT_CHUNKED, LAYOUT_UNITMAJOR, LAYOUT_TILED = 0, 1, 2, 3
QUIRK_NONE, QUIRK_K1_LANE0_SEED, QUIRK_K2_LANE0_CARRY = 0, 1, 2
XORDER_NATURAL, XORDER_K2_LEGACY = 0, 1

OK = 0
ERR_TIMEOUT = -6


class RPTCError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().rptc_strerror(status).decode()
        extra = ""
        if status == -5:
            extra = f" (cudaError {lib().rptc_last_cuda_error()})"
        super().__init__(f"{where}: {msg}{extra} [status {status}]")


class Format(ctypes.Structure):
    """Mirror of `rptc_format`."""
    _fields_ = [("code", ctypes.c_int32), ("K", ctypes.c_int32), ("L", ctypes.c_int32), ("S", ctypes.c_int32),
                ("layout", ctypes.c_int32), ("quirk", ctypes.c_int32)]

    def __init__(self, code=CODE_HASH, K=2, L=16, S=8, layout=LAYOUT_TILED, quirk=QUIRK_NONE):
        super().__init__(code, K, L, S, layout, quirk)

    def replace(self, **kw) -> "Format":
        d = {n: getattr(self, n) for n, _ in self._fields_}
        d.update(kw)
        return Format(**d)

    @property
    def weights_per_unit(self) -> int:
        return 128 // self.K if self.K != 3 else 128   # K=3: per group of three units

    def lut_numel(self) -> int:
        if self.code == CODE_LUT:
            return 1 << self.L
        return 2 << self.S


class GemvInput(ctypes.Structure):
    """Mirror of `rptc_gemv_input`."""
    _fields_ = [("acc", ctypes.c_void_p), ("ld_acc", ctypes.c_int64),
                ("signs_out", ctypes.c_void_p), ("scale_out", ctypes.c_float), ("eps", ctypes.c_float),
                ("signs_in", ctypes.c_void_p), ("h_in", ctypes.c_void_p), ("h_out", ctypes.c_void_p), ("ld_h", ctypes.c_int64),
                ("w_norm", ctypes.c_void_p), ("clear", ctypes.c_void_p), ("clear_count", ctypes.c_int64)]


_lib = None

_SIGS = {
    "rptc_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "rptc_version": (ctypes.c_int, []),
    "rptc_last_cuda_error": (ctypes.c_int, []),
    "rptc_check_device": (ctypes.c_int, []),
    "rptc_device_status": (ctypes.c_int, []),
    "rptc_set_pdl": (None, [ctypes.c_int]),
    "rptc_repack": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                   ctypes.c_int64, ctypes.c_void_p]),
    "rptc_decompress": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(Format), ctypes.c_void_p]),
    "rptc_gemv": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                 ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                 ctypes.POINTER(Format), ctypes.c_void_p]),
    "rptc_gemv_glued": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(GemvInput), ctypes.c_void_p,
                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.POINTER(Format),
                                       ctypes.c_void_p]),
    "rptc_gemv_swiglu": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                        ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.POINTER(Format), ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_void_p]),
    "rptc_gemv_finish": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "rptc_gemv_f16_static": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                            ctypes.c_int, ctypes.POINTER(Format), ctypes.c_void_p]),
    "rptc_gemm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                 ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                 ctypes.POINTER(Format), ctypes.c_void_p]),
    "rptc_hadamard": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                     ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]),
    "rptc_swiglu_hadamard_f16": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                                                ctypes.c_float, ctypes.c_void_p]),
    "rptc_swiglu_hadamard": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                            ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                                            ctypes.c_float, ctypes.c_int, ctypes.c_void_p]),
    "rptc_rmsnorm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                    ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p]),
    "rptc_rope_cache": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                       ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                       ctypes.c_void_p]),
    "rptc_attn_decode": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]),
    "rptc_qkv_attn_decode": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p,
                                            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]),
    "rptc_finish_norm_hadamard": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p,
                                                 ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int,
                                                 ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]),
    "rptc_qkv_finish": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]),
    "rptc_dense_gemv": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]),
    "rptc_peer_alloc": (ctypes.c_int, [ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]),
    "rptc_peer_free": (ctypes.c_int, [ctypes.c_void_p]),
    "rptc_peer_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "rptc_peer_import": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "rptc_peer_close": (ctypes.c_int, [ctypes.c_void_p]),
    "rptc_peer_finish": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64,
                                        ctypes.c_void_p]),
    "rptc_embed": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                  ctypes.c_int64, ctypes.c_void_p]),
    "rptc_viterbi_workspace_bytes": (ctypes.c_int64, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int]),
    "rptc_viterbi_encode": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                           ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
    "rptc_rope_cache_prompt": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                              ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                              ctypes.c_void_p]),
    "rptc_next_token": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "rptc_embed_mailbox": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                          ctypes.c_void_p]),
}


def lib() -> ctypes.CDLL:
    """Loads the C-ABI library once.  Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python let-it-slide_b200/build.py` "
                              "(there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            if hasattr(L, name):
                fn = getattr(L, name)
                fn.restype = res
                fn.argtypes = args
        _lib = L
    return _lib


def exported_symbols() -> list[str]:
    return list(_SIGS)


def check(status: int, where: str) -> None:
    if status != OK:
        raise RPTCError(status, where)


def stream_ptr(stream: torch.cuda.Stream | None = None) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()
