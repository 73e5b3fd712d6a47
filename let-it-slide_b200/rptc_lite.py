"""`rptc_lite` with the reference's function names (rptc_lite.py:12,19,63), in torch over the B200 library.

    index_fn(x, L, S)
    quantize(alphabet, L, S, R, importance, samples) -> (quantized, expected_loss)
    dequantize(alphabet, L, S, R, quantized) -> dequantized [T, 2]

`quantize` is the offline Viterbi encoder (rptc_lite.py:19-60); `dequantize` is the hot path and runs
on the CUDA decompress kernel (code LITE), so it needs CUDA tensors.  The codebook is fp16 on the
device; results are the fp16-rounded alphabet rows cast back to the alphabet's dtype.
"""
from __future__ import annotations

import torch

from rptc import pack_symbols
from rptc_b200 import CODE_LITE, LAYOUT_ROWMAJOR, Format, ops


def index_fn(x: torch.Tensor, L: int, S: int) -> torch.Tensor:
    """rptc_lite.py:12-16 with 32-bit wrap-around."""
    x = x.to(torch.int32)
    x = x * (2 * x + 1)
    x = x ^ (x >> (L - S))
    return x & ((1 << S) - 1)


def quantize(alphabet: torch.Tensor, L: int, S: int, R: int, importance: torch.Tensor, samples: torch.Tensor):
    """rptc_lite.py:19-60 for one sequence: samples, importance [length, V]."""
    length, V = samples.shape
    assert importance.shape == samples.shape
    dev = samples.device
    M = 1 << L
    permuted = alphabet[index_fn(torch.arange(M, device=dev), L, S).long()]              # [M, V]
    rho = torch.full((M,), float("inf"), dtype=alphabet.dtype, device=dev)
    rho[0] = 0
    back = torch.empty((length, M >> R), dtype=torch.int16, device=dev)
    for index in range(length):
        best, msb = rho.view(1 << R, M >> R).min(dim=0)                                  # rptc_lite.py:35-36
        back[index] = msb.to(torch.int16)
        loss = (importance[index] * (samples[index] - permuted) ** 2).sum(dim=-1)
        rho = best.repeat_interleave(1 << R) + loss
    expected_loss, state = rho.min(dim=0)
    quantized = torch.empty(length, dtype=torch.int32, device=dev)
    for index in range(length - 1, -1, -1):                                              # rptc_lite.py:49-52
        quantized[index] = (state & ((1 << R) - 1)).to(torch.int32)
        prefix = state >> R
        state = (back[index, prefix].to(torch.int64) << (L - R)) | prefix
    return quantized, expected_loss


def dequantize(alphabet: torch.Tensor, L: int, S: int, R: int, quantized: torch.Tensor) -> torch.Tensor:
    """rptc_lite.py:63-73 on the GPU: `quantized` [T] (or [rows, T]) symbols of R bits -> [T, 2] (or [rows, T, 2])."""
    if not quantized.is_cuda:
        raise RuntimeError("dequantize runs on the CUDA kernels: pass CUDA tensors")
    if alphabet.shape[1] != 2 or R not in (4, 8):
        raise NotImplementedError("the kernels implement V = 2 with R = 4 or 8 bits per step")
    single = quantized.dim() == 1
    q = quantized[None, :] if single else quantized
    rows, T = q.shape
    pad_rows = -(-rows // 32) * 32
    words = pack_symbols(q, R)
    if pad_rows != rows:
        words = torch.cat([words, words.new_zeros((pad_rows - rows, words.shape[1]))])
    K = R // 2
    n = words.shape[1] * 32 // K
    out = ops.decompress(words.contiguous(), alphabet.to(device=q.device, dtype=torch.float16).contiguous().reshape(-1), pad_rows, n,
                         Format(CODE_LITE, K, L, S, LAYOUT_ROWMAJOR))
    out = out[:rows, : 2 * T].reshape(rows, T, 2).to(alphabet.dtype)
    return out[0] if single else out
