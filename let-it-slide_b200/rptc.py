"""`rptc` with the reference's function names (rptc.py:13,74), in torch over the B200 library.

    quantize(permuted_alphabet, corrections, samples, diag_only=True) -> (quantized, expected_loss)
    dequantize(permuted_alphabet, quantized) -> dequantized

`quantize` is the Viterbi encoder of rptc.py:13-71 (state = last L bits, 2 bits per step, start
state 0, first-minimum tie break); it is the offline half: CUDA fp32 tensors take the CUDA encoder
(csrc/viterbi.cu), anything else a torch restatement of the same recurrence.
`dequantize` is the decoder of rptc.py:74-85 and is the hot path: it packs the symbols into the
MSB-first bitstream the kernels read and calls the CUDA decompress kernel, so it needs CUDA tensors
(there is no CPU decode path in this package).  The codebook is held in fp16 on the device, as in
the reference's kernels (inference.cu:114-117): `dequantize` returns the fp16-rounded alphabet
entries, cast back to the alphabet's dtype.
"""
from __future__ import annotations

import torch

from rptc_b200 import CODE_LUT, LAYOUT_ROWMAJOR, Format, ops


def quantize_rows(permuted_alphabet: torch.Tensor, weights: torch.Tensor, samples: torch.Tensor):
    """Batched form of `quantize` with diagonal corrections: samples [B, length], weights [length]
    (the per-position factor sum(corrections[index]**2)).  Returns (symbols int32 [B, length], loss [B])."""
    M = permuted_alphabet.shape[0]
    L = M.bit_length() - 1
    B, length = samples.shape
    dev, dt = samples.device, permuted_alphabet.dtype
    if samples.is_cuda and dt == torch.float32 and 4 <= L <= 16:
        # the CUDA encoder: same recurrence, ties and fp32 arithmetic, one launch per position for a batch of rows
        return ops.viterbi_encode(permuted_alphabet, weights, samples)
    rho = torch.full((B, M), float("inf"), dtype=dt, device=dev)
    rho[:, 0] = 0                                              # initial state is zero (rptc.py:57-58)
    back = torch.empty((length, B, M >> 2), dtype=torch.uint8, device=dev)
    for index in range(length):
        cand = rho.view(B, 4, M >> 2)                          # cand[b, d, p] = rho[(d << (L-2)) | p]  (rptc.py:27-30)
        best, disc = cand.min(dim=1)                           # first minimum, like jnp.argmin
        back[index] = disc.to(torch.uint8)
        loss = weights[index] * (samples[:, index, None] - permuted_alphabet[None, :]) ** 2
        rho = best.repeat_interleave(4, dim=1) + loss          # rptc.py:52
    expected_loss, state = rho.min(dim=1)
    quantized = torch.empty((B, length), dtype=torch.int32, device=dev)
    rows = torch.arange(B, device=dev)
    for index in range(length - 1, -1, -1):                    # rptc.py:62-68
        quantized[:, index] = (state & 3).to(torch.int32)
        prefix = state >> 2
        state = (back[index, rows, prefix].to(torch.int64) << (L - 2)) | prefix
    return quantized, expected_loss


def quantize(permuted_alphabet: torch.Tensor, corrections: torch.Tensor, samples: torch.Tensor, diag_only: bool = True):
    """rptc.py:13-71 for one row.  Only the diagonal form (the one every call site of the reference uses,
    quantize_hf.py:165 and rptc.py:95) is implemented."""
    if not diag_only:
        raise NotImplementedError("the reference's non-diagonal correction walk (rptc.py:38-50) is not implemented")
    length = samples.shape[0]
    assert samples.dim() == 1 and corrections.shape == (length, length)
    weights = (corrections ** 2).sum(dim=1)
    q, loss = quantize_rows(permuted_alphabet, weights, samples[None, :])
    return q[0], loss[0]


def pack_symbols(quantized: torch.Tensor, bits: int = 2) -> torch.Tensor:
    """[rows, length] symbols -> ROWMAJOR int32 words, MSB first, rows padded to whole 128-bit units."""
    rows, length = quantized.shape
    per = 32 // bits
    assert 32 % bits == 0
    n_words = -(-length // (4 * per)) * 4
    sym = torch.zeros((rows, n_words * per), dtype=torch.int64, device=quantized.device)
    sym[:, :length] = quantized.to(torch.int64)
    shifts = (bits * (per - 1 - torch.arange(per, device=quantized.device))).to(torch.int64)
    words = (sym.view(rows, n_words, per) << shifts).sum(dim=2)
    return (words & 0xFFFFFFFF).to(torch.int64).where(words < 2**31, words - 2**32).to(torch.int32)


def dequantize(permuted_alphabet: torch.Tensor, quantized: torch.Tensor) -> torch.Tensor:
    """rptc.py:74-85 on the GPU: `quantized` [length] or [rows, length] symbols in 0..3."""
    if not quantized.is_cuda:
        raise RuntimeError("dequantize runs on the CUDA kernels: pass CUDA tensors")
    single = quantized.dim() == 1
    q = quantized[None, :] if single else quantized
    rows, length = q.shape
    L = permuted_alphabet.shape[0].bit_length() - 1
    pad_rows = -(-rows // 32) * 32
    words = pack_symbols(q, 2)
    if pad_rows != rows:
        words = torch.cat([words, words.new_zeros((pad_rows - rows, words.shape[1]))])
    n = words.shape[1] * 16
    out = ops.decompress(words.contiguous(), permuted_alphabet.to(device=q.device, dtype=torch.float16).contiguous(), pad_rows, n,
                         Format(CODE_LUT, 2, L, 0, LAYOUT_ROWMAJOR))
    out = out[:rows, :length].to(permuted_alphabet.dtype)
    return out[0] if single else out
