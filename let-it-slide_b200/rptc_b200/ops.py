"""Tensor-level front end of the C ABI: thin argument checking, no arithmetic of its own."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import (CODE_HASH, CODE_LITE, CODE_LUT, LAYOUT_CHUNKED, LAYOUT_ROWMAJOR, LAYOUT_TILED, LAYOUT_UNITMAJOR, XORDER_NATURAL,
                   Format, check, lib, ptr, stream_ptr)


def _cuda_contig(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")


def _ld(t: torch.Tensor, width: int) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(width, t.stride(0))


def units_per_row(n: int, K: int) -> int:
    if (n * K) % 128:
        raise RuntimeError(f"n*K = {n * K} bits per row is not a whole number of 128-bit units")
    return n * K // 128


def codes_shape(m: int, n: int, K: int, layout: int) -> tuple[int, ...]:
    nu = units_per_row(n, K)
    if layout == LAYOUT_ROWMAJOR:
        return (m, nu * 4)
    if layout == LAYOUT_CHUNKED:
        return (nu // 32, m, 128)
    if layout == LAYOUT_UNITMAJOR:
        return (nu, m, 4)
    return (m // 32, nu, 32, 4)


def repack(codes: torch.Tensor, src_layout: int, dst_layout: int, m: int, n_units: int) -> torch.Tensor:
    """Packed codes in `src_layout` -> a new tensor in `dst_layout` (rptc_repack)."""
    _cuda_contig(codes, "codes", torch.int32)
    if codes.numel() != m * n_units * 4:
        raise RuntimeError("codes has the wrong number of elements")
    if dst_layout == LAYOUT_ROWMAJOR:
        shape = (m, n_units * 4)
    elif dst_layout == LAYOUT_CHUNKED:
        shape = (n_units // 32, m, 128)
    elif dst_layout == LAYOUT_UNITMAJOR:
        shape = (n_units, m, 4)
    else:
        shape = (m // 32, n_units, 32, 4)
    out = torch.empty(shape, dtype=torch.int32, device=codes.device)
    with torch.cuda.device(codes.device):
        check(lib().rptc_repack(ptr(codes), src_layout, ptr(out), dst_layout, m, n_units, stream_ptr()), "rptc_repack")
    return out


def decompress(codes: torch.Tensor, lut: torch.Tensor, m: int, n: int, fmt: Format, out: torch.Tensor | None = None,
               carry_in: torch.Tensor | None = None) -> torch.Tensor:
    """Packed codes -> dense fp16 [m, n] (rptc_decompress)."""
    _cuda_contig(codes, "codes", torch.int32)
    _cuda_contig(lut, "lut", torch.float16)
    if lut.numel() != fmt.lut_numel():
        raise RuntimeError(f"lut must have {fmt.lut_numel()} elements, got {lut.numel()}")
    if codes.numel() * 32 != m * n * fmt.K:
        raise RuntimeError("codes has the wrong number of elements for m, n, K")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float16, device=codes.device)
    else:
        if not out.is_cuda or out.dtype != torch.float16 or out.dim() != 2 or out.shape != (m, n) or out.stride(1) != 1:
            raise RuntimeError("out must be a CUDA fp16 [m, n] tensor with unit column stride")
    if carry_in is not None:
        _cuda_contig(carry_in, "carry_in", torch.int32)
    with torch.cuda.device(codes.device):
        check(lib().rptc_decompress(ptr(codes), ptr(lut), ptr(carry_in), ptr(out), out.stride(0), m, n, ctypes.byref(fmt),
                                    stream_ptr()), "rptc_decompress")
    return out


def gemv_acc(codes: torch.Tensor, lut: torch.Tensor, x: torch.Tensor, acc: torch.Tensor, m: int, n: int, fmt: Format,
             x_order: int = XORDER_NATURAL, carry_in: torch.Tensor | None = None) -> None:
    """acc[b, :m] += W x[b]  (fp32 accumulator; rptc_gemv).  x: fp16 [b, n] or [n]."""
    _cuda_contig(codes, "codes", torch.int32)
    _cuda_contig(lut, "lut", torch.float16)
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if acc.dim() == 1:
        acc = acc.unsqueeze(0)
    if not x.is_cuda or x.dtype != torch.float16 or x.stride(1) != 1 or x.shape[1] != n:
        raise RuntimeError("x must be a CUDA fp16 [batch, n] tensor with unit column stride")
    if not acc.is_cuda or acc.dtype != torch.float32 or acc.stride(1) != 1 or acc.shape[1] < m or acc.shape[0] != x.shape[0]:
        raise RuntimeError("acc must be a CUDA fp32 [batch, >=m] tensor")
    if codes.numel() * 32 != m * n * fmt.K:
        raise RuntimeError("codes has the wrong number of elements for m, n, K")
    if lut.numel() != fmt.lut_numel():
        raise RuntimeError(f"lut must have {fmt.lut_numel()} elements, got {lut.numel()}")
    with torch.cuda.device(codes.device):
        check(lib().rptc_gemv(ptr(codes), ptr(lut), ptr(carry_in), ptr(x), x.stride(0) if x.shape[0] > 1 else max(n, x.stride(0)),
                              ptr(acc), acc.stride(0) if acc.shape[0] > 1 else max(m, acc.stride(0)), m, n, x.shape[0],
                              x_order, ctypes.byref(fmt), stream_ptr()), "rptc_gemv")


def gemv_norm_input(codes: torch.Tensor, lut: torch.Tensor, acc: torch.Tensor, m: int, n: int, fmt: Format, rows: int,
                    prev_acc: torch.Tensor | None, signs_out: torch.Tensor | None, scale_out: float, h_in: torch.Tensor,
                    h_out: torch.Tensor, w_norm: torch.Tensor, eps: float, signs_in: torch.Tensor | None,
                    clear: torch.Tensor | None = None, carry_in: torch.Tensor | None = None) -> None:
    """acc += W x with x = H(s_in * rmsnorm(h_in + s_out * H(prev_acc) * scale_out) * w_norm), computed inside the
    launch; the updated residual goes to h_out (rptc_gemv_glued).  `clear` is zeroed by the launch."""
    from ._lib import GemvInput
    d = GemvInput(ptr(prev_acc), 0 if prev_acc is None else _ld(prev_acc, n), ptr(signs_out), scale_out, eps,
                  ptr(signs_in), ptr(h_in), ptr(h_out), _ld(h_in, n), ptr(w_norm), ptr(clear), 0 if clear is None else clear.numel())
    with torch.cuda.device(codes.device):
        check(lib().rptc_gemv_glued(ptr(codes), ptr(lut), ptr(carry_in), ctypes.byref(d), ptr(acc), _ld(acc, m), m, n, rows,
                                    ctypes.byref(fmt), stream_ptr()), "rptc_gemv_glued")


def gemv_swiglu_input(codes: torch.Tensor, lut: torch.Tensor, acc: torch.Tensor, m: int, n: int, fmt: Format, rows: int,
                      prev_acc: torch.Tensor, signs_out: torch.Tensor | None, scale_out: float, signs_in: torch.Tensor | None,
                      block: int, clear: torch.Tensor | None = None, carry_in: torch.Tensor | None = None) -> None:
    """acc += W x with x = H(s_in * silu(g) * u), (g | u) = s_out * H(prev_acc) * scale_out, made inside the launch
    block by block (rptc_gemv_swiglu).  `clear` is zeroed by the launch."""
    with torch.cuda.device(codes.device):
        check(lib().rptc_gemv_swiglu(ptr(codes), ptr(lut), ptr(carry_in), ptr(prev_acc), _ld(prev_acc, 2 * n), ptr(signs_out), scale_out,
                                     ptr(signs_in), block, ptr(acc), _ld(acc, m), m, n, rows, ctypes.byref(fmt), ptr(clear),
                                     0 if clear is None else clear.numel(), stream_ptr()), "rptc_gemv_swiglu")


def gemv_finish(acc: torch.Tensor, y: torch.Tensor, m: int, scale: float = 1.0, accumulate: bool = False,
                clear: bool = True) -> None:
    """y = fp16(scale * acc) (+ y); optionally zero acc (rptc_gemv_finish)."""
    if acc.dim() == 1:
        acc = acc.unsqueeze(0)
    if y.dim() == 1:
        y = y.unsqueeze(0)
    with torch.cuda.device(acc.device):
        check(lib().rptc_gemv_finish(ptr(acc), acc.stride(0) if acc.shape[0] > 1 else max(m, acc.stride(0)), ptr(y),
                                     y.stride(0) if y.shape[0] > 1 else max(m, y.stride(0)), m, acc.shape[0], scale,
                                     int(accumulate), int(clear), stream_ptr()), "rptc_gemv_finish")


def gemv(codes: torch.Tensor, lut: torch.Tensor, x: torch.Tensor, m: int, n: int, fmt: Format,
         x_order: int = XORDER_NATURAL, carry_in: torch.Tensor | None = None) -> torch.Tensor:
    """Convenience: allocate a zeroed fp32 accumulator, run the fused matvec, return fp16 [b, m]."""
    xb = x.unsqueeze(0) if x.dim() == 1 else x
    acc = torch.zeros((xb.shape[0], m), dtype=torch.float32, device=x.device)
    gemv_acc(codes, lut, xb, acc, m, n, fmt, x_order, carry_in)
    y = torch.empty((xb.shape[0], m), dtype=torch.float16, device=x.device)
    gemv_finish(acc, y, m, clear=False)
    return y[0] if x.dim() == 1 else y


def gemm(codes: torch.Tensor, lut: torch.Tensor, x: torch.Tensor, m: int, n: int, fmt: Format,
         out: torch.Tensor | None = None, carry_in: torch.Tensor | None = None) -> torch.Tensor:
    """y[t] = W x[t] for a block of tokens on the tensor cores (rptc_gemm).  x: fp16 [tokens, n]."""
    _cuda_contig(codes, "codes", torch.int32)
    _cuda_contig(lut, "lut", torch.float16)
    if not x.is_cuda or x.dtype != torch.float16 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != n:
        raise RuntimeError("x must be a CUDA fp16 [tokens, n] tensor with unit column stride")
    if out is None:
        out = torch.empty((x.shape[0], m), dtype=torch.float16, device=x.device)
    with torch.cuda.device(codes.device):
        check(lib().rptc_gemm(ptr(codes), ptr(lut), ptr(carry_in), ptr(x), x.stride(0), ptr(out), out.stride(0), m, n,
                              x.shape[0], ctypes.byref(fmt), stream_ptr()), "rptc_gemm")
    return out


def hadamard(x: torch.Tensor, signs: torch.Tensor | None, block: int, transpose: bool = False, scale: float = 1.0,
             out: torch.Tensor | None = None, clear_in: bool = False, residual: torch.Tensor | None = None) -> torch.Tensor:
    """Block-diagonal randomized Hadamard transform along the last axis (rptc_hadamard).

    x: fp16 or fp32 [rows, n]; result fp16 [rows, n] (+ residual)."""
    squeeze = x.dim() == 1
    if squeeze:
        x = x.unsqueeze(0)
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1 or x.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("x must be a CUDA fp16/fp32 [rows, n] tensor with unit column stride")
    rows, n = x.shape
    if out is None:
        out = torch.empty((rows, n), dtype=torch.float16, device=x.device)
    if signs is not None:
        _cuda_contig(signs, "signs", torch.float16)
    if residual is not None and residual.dim() == 1:
        residual = residual.unsqueeze(0)
    with torch.cuda.device(x.device):
        check(lib().rptc_hadamard(ptr(x), int(x.dtype == torch.float32), _ld(x, n), ptr(out), _ld(out, n), ptr(signs),
                                  ptr(residual), 0 if residual is None else _ld(residual, n), rows, n, block, int(transpose),
                                  scale, int(clear_in), stream_ptr()), "rptc_hadamard")
    return out[0] if squeeze else out


def swiglu_hadamard(acc: torch.Tensor, out: torch.Tensor, signs_out: torch.Tensor | None, signs_in: torch.Tensor | None,
                    n: int, block: int, scale_out: float, scale_in: float = 1.0, clear: bool = True) -> torch.Tensor:
    """Fused gated-MLP middle (rptc_swiglu_hadamard): acc fp32 [rows, 2n] -> out fp16 [rows, n]."""
    with torch.cuda.device(acc.device):
        check(lib().rptc_swiglu_hadamard(ptr(acc), _ld(acc, 2 * n), ptr(out), _ld(out, n), ptr(signs_out), ptr(signs_in),
                                         acc.shape[0], n, block, scale_out, scale_in, int(clear), stream_ptr()),
              "rptc_swiglu_hadamard")
    return out


def swiglu_hadamard_f16(gate_up: torch.Tensor, out: torch.Tensor, signs_out: torch.Tensor | None, signs_in: torch.Tensor | None,
                        n: int, block: int, scale_out: float, scale_in: float = 1.0) -> torch.Tensor:
    """Fused gated-MLP middle from the fp16 output of a matrix product (rptc_swiglu_hadamard_f16):
    gate_up fp16 [rows, 2n] -> out fp16 [rows, n]."""
    with torch.cuda.device(gate_up.device):
        check(lib().rptc_swiglu_hadamard_f16(ptr(gate_up), _ld(gate_up, 2 * n), ptr(out), _ld(out, n), ptr(signs_out), ptr(signs_in),
                                             gate_up.shape[0], n, block, scale_out, scale_in, stream_ptr()),
              "rptc_swiglu_hadamard_f16")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float) -> torch.Tensor:
    rows, n = x.shape
    with torch.cuda.device(x.device):
        check(lib().rptc_rmsnorm(ptr(x), _ld(x, n), ptr(w), ptr(out), _ld(out, n), rows, n, eps, stream_ptr()), "rptc_rmsnorm")
    return out


def rope_cache(qkv: torch.Tensor, pos: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, hq: int, hkv: int, d: int,
               theta: float) -> None:
    rows = qkv.shape[0]
    with torch.cuda.device(qkv.device):
        check(lib().rptc_rope_cache(ptr(qkv), _ld(qkv, qkv.shape[1]), ptr(pos), ptr(kcache), ptr(vcache), rows, hq, hkv, d,
                                    kcache.shape[1], theta, stream_ptr()), "rptc_rope_cache")


def rope_cache_prompt(qkv: torch.Tensor, rows: int, tokens: int, kcache: torch.Tensor, vcache: torch.Tensor, hq: int, hkv: int, d: int,
                      theta: float) -> None:
    """RoPE of q (in place) and k, and the cache writes of k and v, for a whole prompt (rptc_rope_cache_prompt):
    qkv fp16 [rows * tokens, (hq + 2 hkv) d]."""
    with torch.cuda.device(qkv.device):
        check(lib().rptc_rope_cache_prompt(ptr(qkv), _ld(qkv, qkv.shape[1]), rows, tokens, ptr(kcache), ptr(vcache), hq, hkv, d,
                                           kcache.shape[1], theta, stream_ptr()), "rptc_rope_cache_prompt")


def attn_decode(qkv: torch.Tensor, pos: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, out: torch.Tensor, hq: int,
                hkv: int, d: int, signs_in: torch.Tensor | None = None) -> torch.Tensor:
    rows = qkv.shape[0]
    with torch.cuda.device(qkv.device):
        check(lib().rptc_attn_decode(ptr(qkv), _ld(qkv, qkv.shape[1]), ptr(pos), ptr(kcache), ptr(vcache), ptr(out),
                                     _ld(out, out.shape[1]), rows, hq, hkv, d, kcache.shape[1], d ** -0.5, ptr(signs_in),
                                     stream_ptr()), "rptc_attn_decode")
    return out


def qkv_attn_decode(acc: torch.Tensor, signs_out: torch.Tensor | None, scale_out: float, pos: torch.Tensor, kcache: torch.Tensor,
                    vcache: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, theta: float,
                    signs_in: torch.Tensor | None) -> torch.Tensor:
    """Output transform of the fused qkv layer + RoPE + KV append + attention (+ per-head input transform of the
    output projection) in one launch (rptc_qkv_attn_decode)."""
    rows = acc.shape[0]
    with torch.cuda.device(acc.device):
        check(lib().rptc_qkv_attn_decode(ptr(acc), _ld(acc, acc.shape[1]), ptr(signs_out), scale_out, ptr(pos), ptr(kcache),
                                         ptr(vcache), ptr(out), _ld(out, out.shape[1]), rows, heads, kv_heads, kcache.shape[1], theta,
                                         ptr(signs_in), stream_ptr()), "rptc_qkv_attn_decode")
    return out


def finish_norm_hadamard(acc: torch.Tensor | None, signs_out: torch.Tensor | None, scale_out: float, h: torch.Tensor,
                         w_norm: torch.Tensor, eps: float, signs_in: torch.Tensor | None, transform_in: bool,
                         out: torch.Tensor) -> torch.Tensor:
    """h += output transform of acc; out = input transform of rmsnorm(h) (rptc_finish_norm_hadamard)."""
    rows, n = h.shape
    with torch.cuda.device(h.device):
        check(lib().rptc_finish_norm_hadamard(ptr(acc), 0 if acc is None else _ld(acc, n), ptr(signs_out), scale_out, ptr(h),
                                              _ld(h, n), ptr(w_norm), eps, ptr(signs_in), int(transform_in), ptr(out),
                                              _ld(out, n), rows, n, stream_ptr()), "rptc_finish_norm_hadamard")
    return out


def qkv_finish(acc: torch.Tensor, signs_out: torch.Tensor | None, scale: float, q_out: torch.Tensor, kcache: torch.Tensor,
               vcache: torch.Tensor, pos: torch.Tensor, hq: int, hkv: int, block: int, theta: float) -> None:
    """Output transform of the fused qkv layer + RoPE + KV-cache append (rptc_qkv_finish)."""
    rows = acc.shape[0]
    with torch.cuda.device(acc.device):
        check(lib().rptc_qkv_finish(ptr(acc), _ld(acc, acc.shape[1]), ptr(signs_out), scale, ptr(q_out), _ld(q_out, q_out.shape[1]),
                                    ptr(kcache), ptr(vcache), ptr(pos), rows, hq, hkv, kcache.shape[1], block, theta,
                                    stream_ptr()), "rptc_qkv_finish")


def dense_gemv(W: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """y[b] = W x[b] for a dense fp16 W [m, n] (rptc_dense_gemv)."""
    squeeze = x.dim() == 1
    if squeeze:
        x = x.unsqueeze(0)
    m, n = W.shape
    if out is None:
        out = torch.empty((x.shape[0], m), dtype=torch.float16, device=x.device)
    o2 = out.unsqueeze(0) if out.dim() == 1 else out
    with torch.cuda.device(W.device):
        for b0 in range(0, x.shape[0], 8):              # the kernel takes up to eight activation rows per launch
            xb, ob = x[b0:b0 + 8], o2[b0:b0 + 8]
            check(lib().rptc_dense_gemv(ptr(W), W.stride(0), ptr(xb), _ld(xb, n), ptr(ob), _ld(ob, m), m, n, xb.shape[0], stream_ptr()),
                  "rptc_dense_gemv")
    return out[0] if squeeze and out.dim() == 2 else out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    with torch.cuda.device(table.device):
        check(lib().rptc_embed(ptr(table), ptr(ids), ptr(out), _ld(out, table.shape[1]), ids.shape[0], table.shape[1],
                               stream_ptr()), "rptc_embed")
    return out


def embed_mailbox(table: torch.Tensor, slots: torch.Tensor, steps_done: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
                  timeout_ms: int = 2000) -> None:
    """Embedding rows of the ids the host posts in `slots` (pinned int64: sequence << 32 | id); waits for them, bounded
    (rptc_embed_mailbox)."""
    if not slots.is_pinned() or slots.dtype != torch.int64 or steps_done.dtype != torch.int32:
        raise RuntimeError("slots must be a pinned int64 host tensor and steps_done an int32 device tensor")
    with torch.cuda.device(table.device):
        check(lib().rptc_embed_mailbox(ptr(table), ptr(slots), ptr(steps_done), ptr(ids), ptr(out), _ld(out, table.shape[1]),
                                       ids.shape[0], table.shape[1], table.shape[0], timeout_ms, stream_ptr()), "rptc_embed_mailbox")


def next_token(logits: torch.Tensor, next_ids: torch.Tensor, ids: torch.Tensor | None = None, pos: torch.Tensor | None = None,
               mirror: torch.Tensor | None = None, steps_done: torch.Tensor | None = None) -> None:
    """Greedy choice + feedback + position bump in one launch (rptc_next_token).  `mirror`: pinned host int64."""
    rows, n = logits.shape
    if next_ids.dtype != torch.int64 or (mirror is not None and (mirror.dtype != torch.int64 or not mirror.is_pinned())):
        raise RuntimeError("next_ids must be int64 and mirror a pinned int64 host tensor")
    with torch.cuda.device(logits.device):
        check(lib().rptc_next_token(ptr(logits), _ld(logits, n), rows, n, ptr(next_ids), ptr(ids), ptr(pos), ptr(mirror),
                                    ptr(steps_done), stream_ptr()), "rptc_next_token")


def viterbi_encode(alphabet: torch.Tensor, pos_weight: torch.Tensor, samples: torch.Tensor, workspace_limit: int = 12 << 30):
    """Code-A trellis encoder on the GPU (rptc_viterbi_encode): samples fp32 [rows, n] -> (symbols int32 [rows, n],
    loss fp32 [rows]).  Rows go through in batches sized so that the survivor memory stays under `workspace_limit`."""
    M = alphabet.numel()
    L = M.bit_length() - 1
    if M != 1 << L:
        raise RuntimeError("the alphabet must have 2^L entries")
    alphabet = alphabet.to(torch.float32).contiguous()
    pos_weight = pos_weight.to(torch.float32).contiguous()
    samples = samples.to(torch.float32).contiguous()
    rows, n = samples.shape
    symbols = torch.empty((rows, n), dtype=torch.int32, device=samples.device)
    loss = torch.empty(rows, dtype=torch.float32, device=samples.device)
    per_row = lib().rptc_viterbi_workspace_bytes(1, n, L)
    batch = max(1, min(rows, 128, workspace_limit // per_row))
    with torch.cuda.device(samples.device):
        need = lib().rptc_viterbi_workspace_bytes(batch, n, L)
        ws = torch.empty(need, dtype=torch.uint8, device=samples.device)
        for r0 in range(0, rows, batch):
            r = min(batch, rows - r0)
            check(lib().rptc_viterbi_encode(ptr(alphabet), ptr(pos_weight), ptr(samples[r0:]), n, r, n, L, ptr(symbols[r0:]), n,
                                            ptr(loss[r0:]), ptr(ws), need, stream_ptr()), "rptc_viterbi_encode")
    return symbols, loss


def device_status() -> None:
    """Raises if a kernel reported a timed-out wait since the last call."""
    check(lib().rptc_device_status(), "rptc_device_status")
