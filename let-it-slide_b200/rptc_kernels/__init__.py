"""Drop-in for the reference's `rptc_kernels` torch extension (wrapper.cpp:59-67).

Same seven functions, same argument order, same in-place outputs, same `float` return value
(elapsed milliseconds), same RuntimeError on a bad shape or dtype — on top of the sm_100a library
instead of the reference's kernels.  Differences, all deliberate:
  * work runs on torch's current stream and is timed there (the reference times a private stream,
    and launches the fused kernel on the default stream, inference.cu:131-132,335);
  * a CUDA failure raises instead of calling exit() (inference.cu:32-39);
  * by default the row's stream is decoded self-consistently (rptc.py:74-85).  The reference kernels
    deviate from it at every 32nd 128-bit unit (inference.cu:61-62 and :232);
    `set_reference_quirks(True)` reproduces those deviations bit for bit;
  * `decompress_matvec_t_*` computes the intended product; the reference kernel's inner loop does
    not advance its shift registers (inference_t.cu:125-134) and is not reproduced;
  * the fused matvecs add partial sums into an fp32 accumulator that this module keeps per (device, stream, m): two
    calls on the same stream are ordered by the stream; calls from two host threads that share one stream must be
    serialised by the caller;
  * shape rules are relaxed: n needs to be a multiple of 64 only, except for the chunked layout of
    `decompress_matvec_*`, which is defined in steps of 2048 columns.
"""
from __future__ import annotations

import torch

from rptc_b200 import (CODE_HASH, CODE_LUT, LAYOUT_CHUNKED, LAYOUT_ROWMAJOR, LAYOUT_UNITMAJOR, QUIRK_K1_LANE0_SEED,
                       QUIRK_K2_LANE0_CARRY, QUIRK_NONE, XORDER_K2_LEGACY, XORDER_NATURAL, Format, ops)

_quirks = False
_scratch: dict[tuple[int, int, int], torch.Tensor] = {}


def set_reference_quirks(enable: bool) -> None:
    """Reproduce (True) or not (False, default) the reference kernels' lane-0 deviations."""
    global _quirks
    _quirks = bool(enable)


def _check(t: torch.Tensor, name: str, dtype: torch.dtype, dim: int | None = None) -> None:
    # CHECK_INPUT / TORCH_CHECK of inference.cu:26-28,103-123
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}")
    if dim is not None and t.dim() != dim:
        raise RuntimeError(f"{name} must have {dim} dimensions")


def _acc(device: torch.device, m: int) -> torch.Tensor:
    """fp32 accumulator of the fused matvecs, one per (device, stream, m): calls on different streams share nothing, like
    the reference's functions, which write `out` directly (inference.cu:335-342)."""
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream, m)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.zeros((1, m), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def _timed(fn) -> float:
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    stop.record()
    stop.synchronize()
    return start.elapsed_time(stop)


def matvec(decompressed: torch.Tensor, x: torch.Tensor, out: torch.Tensor) -> float:
    """Dense fp16 matvec out = decompressed @ x.  The reference's tests call it as a bandwidth probe
    (rptc_kernels/tests/test_matvec.py:18) although wrapper.cpp does not export it."""
    _check(decompressed, "decompressed", torch.float16, 2)
    _check(x, "x", torch.float16, 1)
    _check(out, "out", torch.float16, 1)
    if decompressed.shape[1] != x.shape[0] or decompressed.shape[0] != out.shape[0]:
        raise RuntimeError("shapes of decompressed [m, n], x [n] and out [m] do not agree")
    return _timed(lambda: ops.dense_gemv(decompressed, x, out=out))


_ones: dict[tuple[int, int], torch.Tensor] = {}


def rowsum(decompressed: torch.Tensor, out: torch.Tensor) -> float:
    """out[i] = sum_j decompressed[i, j] (rptc_kernels/tests/test_rowsum.py:17; same remark as `matvec`)."""
    _check(decompressed, "decompressed", torch.float16, 2)
    _check(out, "out", torch.float16, 1)
    key = (decompressed.device.index or 0, decompressed.shape[1])
    if key not in _ones:
        _ones[key] = torch.ones(decompressed.shape[1], dtype=torch.float16, device=decompressed.device)
    return _timed(lambda: ops.dense_gemv(decompressed, _ones[key], out=out))


def decompress(compressed: torch.Tensor, codebook: torch.Tensor, out: torch.Tensor) -> float:
    """inference.cu:99-160.  compressed int32 [m, n/16] -> out fp16 [m, n] through codebook fp16 [65536]."""
    _check(compressed, "compressed", torch.int32, 2)
    _check(codebook, "codebook", torch.float16, 1)
    _check(out, "out", torch.float16, 2)
    m, nw = compressed.shape
    if nw % 4:
        raise RuntimeError("compressed.size(1) must be a multiple of 4 (whole 128-bit units)")
    if codebook.shape[0] != 1 << 16:
        raise RuntimeError("codebook must have 65536 entries")
    n = nw * 16
    if tuple(out.shape) != (m, n):
        raise RuntimeError("out must be [m, n]")
    fmt = Format(CODE_LUT, 2, 16, 0, LAYOUT_ROWMAJOR, QUIRK_K1_LANE0_SEED if _quirks else QUIRK_NONE)
    return _timed(lambda: ops.decompress(compressed, codebook, m, n, fmt, out=out))


def _decompress_matvec(S: int, compressed, codebook, x, out) -> float:
    """inference.cu:280-356.  compressed int32 [n/2048, m, 128]; codebook fp16 [2^(S+1)]; x fp16 [n]; out fp16 [m]."""
    _check(compressed, "compressed", torch.int32, 3)
    if compressed.shape[2] != 128:
        raise RuntimeError("compressed.size(2) must be 128")
    iters, m, _ = compressed.shape
    n = iters * 2048
    _check(codebook, "codebook", torch.float16, 1)
    if codebook.shape[0] != 2 << S:
        raise RuntimeError(f"codebook must have {2 << S} entries")
    _check(x, "x", torch.float16, 1)
    if x.shape[0] != n:
        raise RuntimeError("x must have n elements")
    _check(out, "out", torch.float16, 1)
    if out.shape[0] != m:
        raise RuntimeError("out must have m elements")
    if m % 32:
        raise RuntimeError("m must be a multiple of 32")
    fmt = Format(CODE_HASH, 2, 16, S, LAYOUT_CHUNKED, QUIRK_K2_LANE0_CARRY if _quirks else QUIRK_NONE)
    acc = _acc(out.device, m)

    def run():
        acc.zero_()
        ops.gemv_acc(compressed, codebook, x, acc, m, n, fmt, XORDER_K2_LEGACY)
        ops.gemv_finish(acc, out, m, clear=True)

    return _timed(run)


def decompress_matvec_16_6_1(compressed, codebook, x, out) -> float:
    return _decompress_matvec(6, compressed, codebook, x, out)


def decompress_matvec_20_6_1(compressed, codebook, x, out) -> float:
    # the template's L only appears in static_asserts (inference.cu:287-288): same arithmetic as _16_
    return _decompress_matvec(6, compressed, codebook, x, out)


def decompress_matvec_16_8_1(compressed, codebook, x, out) -> float:
    return _decompress_matvec(8, compressed, codebook, x, out)


def decompress_matvec_20_8_1(compressed, codebook, x, out) -> float:
    return _decompress_matvec(8, compressed, codebook, x, out)


def _decompress_matvec_t(L: int, compressed, codebook, x, out) -> float:
    """inference_t.cu:178-256.  compressed int32 laid out [n/64][m][4]; out is accumulated into."""
    _check(compressed, "compressed", torch.int32)
    _check(codebook, "codebook", torch.float16, 1)
    if codebook.shape[0] != 1 << L:
        raise RuntimeError(f"codebook must have {1 << L} entries")
    _check(x, "x", torch.float16, 1)
    _check(out, "out", torch.float16, 1)
    m, n = out.shape[0], x.shape[0]
    if n % 64 or m % 32:
        raise RuntimeError("n must be a multiple of 64 and m of 32")
    if compressed.numel() != m * n // 16:
        raise RuntimeError("compressed must hold m*n/16 words")
    fmt = Format(CODE_LUT, 2, L, 0, LAYOUT_UNITMAJOR, QUIRK_NONE)
    acc = _acc(out.device, m)

    def run():
        acc.zero_()
        ops.gemv_acc(compressed, codebook, x, acc, m, n, fmt, XORDER_NATURAL)
        ops.gemv_finish(acc, out, m, accumulate=True, clear=True)

    return _timed(run)


def decompress_matvec_t_16(compressed, codebook, x, out) -> float:
    return _decompress_matvec_t(16, compressed, codebook, x, out)


def decompress_matvec_t_14(compressed, codebook, x, out) -> float:
    return _decompress_matvec_t(14, compressed, codebook, x, out)
