"""RPTCLinear: a quantised Linear layer over packed trellis codes.

The reference has no nn.Module (rptc.py / rptc_lite.py are function libraries and quantize_hf.py
writes dense fake-quantised weights back, quantize_hf.py:215); this module is what a model holds
when the 2-bit symbols are kept instead.  y = s_out * H_out( scale * W_hat( H_in( s_in * x ) ) ) with
W_hat decoded on the fly from `codes` through `lut`, H the orthonormal block-diagonal Hadamard
transform and s the +-1 sign vectors ("incoherence processing on both sides").
"""
from __future__ import annotations

import math

import torch
from torch import nn

from . import ops
from ._lib import CODE_HASH, CODE_LITE, CODE_LUT, LAYOUT_TILED, Format


def hadamard_block(n: int) -> int:
    """Largest power of two dividing n, capped at 4096."""
    return min(n & (-n), 4096)


def random_signs(n: int, generator: torch.Generator, device) -> torch.Tensor:
    return (torch.randint(0, 2, (n,), generator=generator, device=device, dtype=torch.int32) * 2 - 1).to(torch.float16)


def gaussian_codebook(fmt: Format, generator: torch.Generator, device) -> torch.Tensor:
    """Codebook in the manner of rptc.py:143-146: Gaussian quantiles in a seeded random order
    (code LUT), or N(0,1) pairs (rptc_lite.py:125, codes HASH / LITE)."""
    if fmt.code == CODE_LUT:
        M = 1 << fmt.L
        q = (2 * torch.arange(M, dtype=torch.float64, device=device) + 1) / (2 * M)
        alphabet = math.sqrt(2.0) * torch.erfinv(2 * q - 1)
        perm = torch.randperm(M, generator=generator, device=device)
        return alphabet[perm].to(torch.float16)
    return torch.randn(2 << fmt.S, generator=generator, device=device, dtype=torch.float32).to(torch.float16)


class RPTCLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, fmt: Format, codes: torch.Tensor, lut: torch.Tensor,
                 scale: float = 1.0, signs_in: torch.Tensor | None = None, signs_out: torch.Tensor | None = None,
                 carry_in: torch.Tensor | None = None):
        super().__init__()
        self.in_features, self.out_features, self.fmt, self.scale = in_features, out_features, fmt, float(scale)
        self.block_in, self.block_out = hadamard_block(in_features), hadamard_block(out_features)
        self.register_buffer("codes", codes)
        self.register_buffer("lut", lut)
        self.register_buffer("signs_in", signs_in)
        self.register_buffer("signs_out", signs_out)
        self.register_buffer("carry_in", carry_in)
        self.incoherent = signs_in is not None
        self._acc: dict[int, torch.Tensor] = {}

    # -- construction -------------------------------------------------------------------------------
    @classmethod
    def random(cls, in_features: int, out_features: int, fmt: Format | None = None, scale: float = 0.02, seed: int = 0,
               device="cuda", incoherent: bool = True) -> "RPTCLinear":
        """Random-init layer: every bitstream is a valid trellis path, so uniform random words are a
        valid quantised weight matrix whose decoded entries are ~ iid draws from the codebook."""
        fmt = fmt or Format(CODE_HASH, 2, 16, 8, LAYOUT_TILED)
        g = torch.Generator(device=device).manual_seed(seed)
        shape = ops.codes_shape(out_features, in_features, fmt.K, fmt.layout)
        codes = torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=device, generator=g)
        lut = gaussian_codebook(fmt, g, device)
        si = random_signs(in_features, g, device) if incoherent else None
        so = random_signs(out_features, g, device) if incoherent else None
        return cls(in_features, out_features, fmt, codes, lut, scale, si, so)

    def get_extra_state(self):
        return {"fmt": [self.fmt.code, self.fmt.K, self.fmt.L, self.fmt.S, self.fmt.layout, self.fmt.quirk],
                "in_features": self.in_features, "out_features": self.out_features, "scale": self.scale}

    def set_extra_state(self, state):
        self.fmt = Format(*state["fmt"])
        self.in_features, self.out_features, self.scale = state["in_features"], state["out_features"], state["scale"]

    # -- forward ------------------------------------------------------------------------------------
    def acc_buffer(self, rows: int) -> torch.Tensor:
        buf = self._acc.get(rows)
        if buf is None:
            buf = torch.zeros((rows, self.out_features), dtype=torch.float32, device=self.codes.device)
            self._acc[rows] = buf
        return buf

    def transform_in(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if not self.incoherent:
            return x
        return ops.hadamard(x, self.signs_in, self.block_in, transpose=False, out=out)

    def matvec_acc(self, x_t: torch.Tensor, acc: torch.Tensor) -> None:
        """acc += W_hat x_t for already-transformed activations (fp32, unscaled)."""
        ops.gemv_acc(self.codes, self.lut, x_t, acc, self.out_features, self.in_features, self.fmt, carry_in=self.carry_in)

    def finish(self, acc: torch.Tensor, out: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
        """out = s_out * H(acc) * scale (+ residual); the accumulator is left zeroed for its next use."""
        if self.incoherent:
            return ops.hadamard(acc, self.signs_out, self.block_out, transpose=True, scale=self.scale, out=out, clear_in=True,
                                residual=residual)
        if out is None:
            out = torch.empty(acc.shape, dtype=torch.float16, device=acc.device)
        if residual is not None:
            if out.data_ptr() != residual.data_ptr():
                out.copy_(residual)
            ops.gemv_finish(acc, out, self.out_features, scale=self.scale, accumulate=True, clear=True)
        else:
            ops.gemv_finish(acc, out, self.out_features, scale=self.scale, clear=True)
        return out

    def product_t(self, xt: torch.Tensor) -> torch.Tensor:
        """W_hat xt for already-transformed activations xt fp16 [rows > 8, in]: the tensor-core GEMM, unscaled and
        before the output transform."""
        return ops.gemm(self.codes, self.lut, xt, self.out_features, self.in_features, self.fmt, carry_in=self.carry_in)

    def finish_t(self, y: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Output side of `product_t`: s_out * H(y) * scale (+ residual), fp16."""
        if self.incoherent:
            return ops.hadamard(y, self.signs_out, self.block_out, transpose=True, scale=self.scale, residual=residual)
        y = y * self.scale if self.scale != 1.0 else y
        return y if residual is None else y + residual

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.in_features).to(torch.float16).contiguous()
        rows = x2.shape[0]
        xt = self.transform_in(x2)
        if rows <= 8:
            acc = self.acc_buffer(rows)
            self.matvec_acc(xt, acc)
            y = self.finish(acc)
        else:
            y = ops.gemm(self.codes, self.lut, xt, self.out_features, self.in_features, self.fmt, carry_in=self.carry_in)
            if self.incoherent:
                y = ops.hadamard(y, self.signs_out, self.block_out, transpose=True, scale=self.scale)
            elif self.scale != 1.0:
                y = y * self.scale
        return y.reshape(*shape[:-1], self.out_features)

    # -- reference helpers ----------------------------------------------------------------------------
    def decoded(self) -> torch.Tensor:
        """W_hat as dense fp16 [out, in] (bit-exact decode on the GPU)."""
        return ops.decompress(self.codes, self.lut, self.out_features, self.in_features, self.fmt, carry_in=self.carry_in)

    def effective_weight(self) -> torch.Tensor:
        """The dense fp32 matrix this layer applies: diag(s_out) H (scale * W_hat) H diag(s_in)."""
        w = self.decoded().float() * self.scale
        if not self.incoherent:
            return w

        def had_rows(a: torch.Tensor, block: int) -> torch.Tensor:      # orthonormal H applied along the last axis
            r, n = a.shape
            a = a.reshape(r, n // block, block)
            h = 1
            while h < block:
                a = a.reshape(r, n // block, block // (2 * h), 2, h)
                a = torch.stack((a[..., 0, :] + a[..., 1, :], a[..., 0, :] - a[..., 1, :]), dim=-2)
                a = a.reshape(r, n // block, block)
                h *= 2
            return a.reshape(r, n) / math.sqrt(block)

        w = had_rows(w, self.block_in) * self.signs_in.float()[None, :]                  # W_hat H diag(s_in)
        w = had_rows(w.t().contiguous(), self.block_out).t() * self.signs_out.float()[:, None]
        return w.contiguous()
