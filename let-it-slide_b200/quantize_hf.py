"""`quantize_hf` with the reference's function names (quantize_hf.py:14-169), in torch over the B200 library.

The reference's driver factorises a weight matrix into row/column biases and scales (`factorize`,
quantize_hf.py:77-117), rounds the normalised remainder with the code-A Viterbi encoder using one
quantile alphabet per bank of rows (`round_weights`, :120-156), and writes the DENSE reconstruction back
into the Hugging Face module (`quantize_model`, :188-215).  Here the same steps produce a PACKED layer:

    biases_out, biases_in, scales_out, scales_in, normalized = factorize(W)
    layer = quantize_layer(permute, H, W, shift_register_size)      # -> FactorizedRPTCLinear
    layer.reconstruct()                                             # what the reference stores
    layer(x)                                                        # runs on the packed codes

and `quantize_model` swaps the packed layers into the model in place of its `nn.Linear`s, so a forward pass
decodes the 2-bit codes inside the fused kernels:

    y = scales_out * (W_hat (scales_in * x)) + biases_out * sum(x) + <biases_in, x>

with W_hat the decoded alphabet entries.  The alphabet is held in fp16 on the device, as in the reference's
kernels (inference.cu:114-117); `reconstruct()` uses the same rounded entries.  The encoder is the offline half
and runs wherever its tensors live; the forward pass needs CUDA (there is no CPU decode path in this package).

`permute` stands in for `jax.random.permutation(key, alphabet)`: any callable alphabet -> permuted alphabet
(JAX's threefry stream is not reproduced; a seeded torch permutation is the default).
"""
from __future__ import annotations

import re
from typing import Callable

import torch
from torch import nn

from rptc import pack_symbols, quantize_rows
from rptc_b200 import CODE_LUT, LAYOUT_ROWMAJOR, LAYOUT_TILED, Format, ops

# Hugging Face projection name -> name of the fused layer its statistics are filed under (quantize_hf.py:14-22)
hf_to_fused = {"q": "qkv", "k": "qkv", "v": "qkv", "o": "o", "up": "up", "gate": "up", "down": "down"}

_PROJ = re.compile(r"model\.layers\.(\d+)\.(self_attn\.(\w+)_proj|mlp\.(\w+)_proj)")      # quantize_hf.py:189


def factorize(W: torch.Tensor):
    """W ~ biases_out + biases_in + scales_out * scales_in * normalized: 64 alternating projection steps
    (quantize_hf.py:77-117).  fp32; returns column vectors [m,1], row vectors [1,n] and the normalised matrix."""
    W = W.to(torch.float32)
    m, n = W.shape
    biases_in = torch.zeros((1, n), dtype=W.dtype, device=W.device)
    scales_out = torch.ones((m, 1), dtype=W.dtype, device=W.device)
    scales_in = torch.ones((1, n), dtype=W.dtype, device=W.device)
    biases_out = torch.zeros((m, 1), dtype=W.dtype, device=W.device)
    for _ in range(64):
        biases_out = ((W - biases_in) / scales_in).mean(dim=1, keepdim=True) / (1 / scales_in).mean()
        biases_in = ((W - biases_out) / scales_out).mean(dim=0, keepdim=True) / (1 / scales_out).mean()
        balance = (biases_in.mean() - biases_out.mean()) / 2
        biases_out = biases_out + balance
        biases_in = biases_in - balance
        centred = W - biases_out - biases_in
        scales_out = ((centred / scales_in) ** 2).mean(dim=1, keepdim=True).sqrt()
        scales_in = ((centred / scales_out) ** 2).mean(dim=0, keepdim=True).sqrt()
        balance = torch.exp((scales_in.log().mean() - scales_out.log().mean()) / 2)
        scales_out = scales_out * balance
        scales_in = scales_in / balance
    normalized = (W - biases_out - biases_in) / scales_out / scales_in
    return biases_out, biases_in, scales_out, scales_in, normalized


def megabatch_alphabet(megabatch: torch.Tensor, shift_register_size: int) -> torch.Tensor:
    """2^L evenly spaced quantiles of a bank's values, by linear interpolation of the sorted sample
    (quantize_hf.py:136-140).  Interpolated in float64 and rounded to fp32."""
    M = 1 << shift_register_size
    fp = torch.sort(megabatch.reshape(-1).to(torch.float64)).values
    N = fp.numel()
    x = (2 * torch.arange(M, dtype=torch.float64, device=fp.device) + 1) / 2 / M
    pos = x * N - 0.5                                  # position of x on the sample grid xp[j] = (2j+1)/(2N)
    lo = pos.floor().clamp(0, N - 1).to(torch.int64)
    hi = (lo + 1).clamp(max=N - 1)
    frac = (pos - lo.to(torch.float64)).clamp(0, 1)
    return (fp[lo] + (fp[hi] - fp[lo]) * frac).to(torch.float32)


def seeded_permute(seed: int) -> Callable[[torch.Tensor], torch.Tensor]:
    def permute(alphabet: torch.Tensor) -> torch.Tensor:
        g = torch.Generator().manual_seed(seed)
        return alphabet[torch.randperm(alphabet.numel(), generator=g).to(alphabet.device)]
    return permute


def round_weights(permute, weights: torch.Tensor, importance: torch.Tensor, shift_register_size: int,
                  num_banks: int = 32, batch_size: int = 8):
    """quantize_hf.py:120-156 without the final decode: rows are split into `num_banks` banks, every bank gets
    its own permuted quantile alphabet, and each row is encoded against it.  `importance` is the DIAGONAL of
    the reference's diagonal correction matrix.  Returns (symbols int32 [m, n], alphabets fp32 [num_banks, 2^L])."""
    m, n = weights.shape
    assert m % (num_banks * batch_size) == 0, (m, num_banks, batch_size)
    per_bank = m // num_banks
    pos_weight = importance.to(torch.float32) ** 2           # sum(corrections[index]**2) of a diagonal matrix (rptc.py:21)
    symbols = torch.empty((m, n), dtype=torch.int32, device=weights.device)
    alphabets = []
    for b in range(num_banks):
        rows = slice(b * per_bank, (b + 1) * per_bank)
        alphabet = permute(megabatch_alphabet(weights[rows], shift_register_size))
        alphabets.append(alphabet)
        for r0 in range(rows.start, rows.stop, batch_size):
            q, _ = quantize_rows(alphabet, pos_weight, weights[r0:r0 + batch_size].to(torch.float32))
            symbols[r0:r0 + batch_size] = q
    return symbols, torch.stack(alphabets)


def evaluate_layer(H: torch.Tensor, W: torch.Tensor, recon: torch.Tensor):
    """Relative squared error under four weightings (quantize_hf.py:171-185): Frobenius, full Hessian proxy,
    its diagonal, its row sums."""
    H, W, recon = H.to(torch.float32), W.to(torch.float32), recon.to(torch.float32)
    E = W - recon
    d, rs = torch.diag(H), H.sum(dim=-1)
    frob = (E ** 2).sum() / (W ** 2).sum() ** 0.5
    proxy = ((E @ H) * E).sum() / ((W @ H) * W).sum()
    proxy_diag = ((E * d) * E).sum() / ((W * d) * W).sum()
    proxy_sum = ((E * rs) * E).sum() / ((W * rs) * W).sum()
    return frob, proxy, proxy_diag, proxy_sum


class FactorizedRPTCLinear(nn.Module):
    """A linear layer stored as code-A trellis codes plus the factorisation's biases and scales.

    Rows are split into `num_banks` banks of out_features / num_banks rows with one alphabet each, as the reference's
    round_weights does (quantize_hf.py:120-156; it needs out_features % (num_banks * batch_size) == 0 only).  The
    kernels decode 32 rows at a time, so each bank is stored padded up to a whole number of 32-row blocks with all-zero
    code rows whose outputs are dropped: Llama-2-7B's gate/up projections (11008 rows, 344 per bank at 32 banks) take 11
    blocks per bank."""

    def __init__(self, out_features: int, in_features: int, shift_register_size: int, num_banks: int, bias: bool = False,
                 device=None):
        super().__init__()
        if in_features % 64 or out_features % num_banks:
            raise ValueError("in_features must be a multiple of 64 and out_features a multiple of num_banks")
        self.out_features, self.in_features, self.L, self.num_banks = out_features, in_features, shift_register_size, num_banks
        self.bank_rows = out_features // num_banks                 # rows of W per bank
        self.bank_blocks = -(-self.bank_rows // 32)                # 32-row blocks per bank as stored (last one zero-padded)
        self.fmt = Format(CODE_LUT, 2, shift_register_size, 0, LAYOUT_TILED)
        dev = device
        self.register_buffer("codes", torch.zeros((num_banks * self.bank_blocks, in_features // 64, 32, 4), dtype=torch.int32, device=dev))
        self.register_buffer("alphabets", torch.zeros((num_banks, 1 << shift_register_size), dtype=torch.float16, device=dev))
        self.register_buffer("biases_out", torch.zeros(out_features, dtype=torch.float32, device=dev))
        self.register_buffer("biases_in", torch.zeros(in_features, dtype=torch.float32, device=dev))
        self.register_buffer("scales_out", torch.ones(out_features, dtype=torch.float32, device=dev))
        self.register_buffer("scales_in", torch.ones(in_features, dtype=torch.float32, device=dev))
        self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float32, device=dev) if bias else None)

    @classmethod
    def from_parts(cls, symbols: torch.Tensor, alphabets: torch.Tensor, biases_out, biases_in, scales_out, scales_in,
                   bias: torch.Tensor | None = None) -> "FactorizedRPTCLinear":
        m, n = symbols.shape
        L = alphabets.shape[1].bit_length() - 1
        dev = torch.device("cuda", torch.cuda.current_device())
        self = cls(m, n, L, alphabets.shape[0], bias is not None, device=dev)
        padded = torch.zeros((self.num_banks, self.bank_blocks * 32, n), dtype=symbols.dtype, device=dev)
        padded[:, : self.bank_rows] = symbols.to(dev).reshape(self.num_banks, self.bank_rows, n)
        words = pack_symbols(padded.reshape(-1, n), bits=2)                 # ROWMAJOR, MSB first
        self.codes.copy_(ops.repack(words.contiguous(), LAYOUT_ROWMAJOR, LAYOUT_TILED, padded.shape[0] * padded.shape[1], n // 64))
        self.alphabets.copy_(alphabets.to(dev))
        for name, v in (("biases_out", biases_out), ("biases_in", biases_in), ("scales_out", scales_out), ("scales_in", scales_in)):
            getattr(self, name).copy_(v.reshape(-1).to(dev))
        if bias is not None:
            self.bias.copy_(bias.to(dev))
        return self

    def _bank(self, b: int):
        """(codes of the bank, its alphabet, rows as stored = a multiple of 32, slice of W's rows the bank holds)."""
        rb = self.bank_blocks
        return self.codes[b * rb:(b + 1) * rb], self.alphabets[b], rb * 32, slice(b * self.bank_rows, (b + 1) * self.bank_rows)

    def decoded(self) -> torch.Tensor:
        """W_hat [m, n] fp16: the alphabet entries the codes select."""
        out = torch.empty((self.out_features, self.in_features), dtype=torch.float16, device=self.codes.device)
        for b in range(self.num_banks):
            codes, lut, stored, sl = self._bank(b)
            out[sl] = ops.decompress(codes, lut, stored, self.in_features, self.fmt)[: self.bank_rows]
        return out

    def reconstruct(self) -> torch.Tensor:
        """The dense matrix the reference writes back into the model (quantize_hf.py:166)."""
        return (self.biases_out[:, None] + self.biases_in[None, :]
                + self.scales_out[:, None] * self.scales_in[None, :] * self.decoded().float())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape, dt = x.shape, x.dtype
        x32 = x.reshape(-1, self.in_features).float()
        xs = (x32 * self.scales_in).to(torch.float16).contiguous()
        t = xs.shape[0]
        y = torch.empty((t, self.out_features), dtype=torch.float32, device=x.device)
        for b in range(self.num_banks):
            codes, lut, stored, sl = self._bank(b)
            if t > 8 and stored % 128 == 0:         # the tensor-core GEMM works on 128-row tiles
                y[:, sl] = ops.gemm(codes, lut, xs, stored, self.in_features, self.fmt)[:, : self.bank_rows].float()
            else:
                for t0 in range(0, t, 8):
                    y[t0:t0 + 8, sl] = ops.gemv(codes, lut, xs[t0:t0 + 8], stored, self.in_features, self.fmt)[:, : self.bank_rows].float()
        y = y * self.scales_out + x32.sum(dim=1, keepdim=True) * self.biases_out + (x32 @ self.biases_in)[:, None]
        if self.bias is not None:
            y = y + self.bias
        return y.to(dt).reshape(*shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return f"{self.in_features} -> {self.out_features}, L={self.L}, banks={self.num_banks}"


def quantize_layer(permute, H: torch.Tensor, W: torch.Tensor, shift_register_size: int, num_banks: int = 32,
                   batch_size: int = 8, bias: torch.Tensor | None = None) -> FactorizedRPTCLinear:
    """quantize_hf.py:159-169, returning the packed layer instead of its dense reconstruction."""
    biases_out, biases_in, scales_out, scales_in, normalized = factorize(W)
    importance = torch.diag(H).to(torch.float32) * scales_in.reshape(-1)        # the diagonal of quantize_hf.py:163
    symbols, alphabets = round_weights(permute, normalized, importance, shift_register_size, num_banks, batch_size)
    return FactorizedRPTCLinear.from_parts(symbols, alphabets, biases_out, biases_in, scales_out, scales_in, bias)


def quantize_model(permute, full_model: nn.Module, load_hessian: Callable[[int, str], torch.Tensor], shift_register_size: int,
                   num_banks: int = 32, batch_size: int = 8, report: Callable[[str], None] | None = print) -> dict:
    """quantize_hf.py:188-215: every `self_attn.*_proj` / `mlp.*_proj` of a Hugging Face Llama is quantised with the
    Hessian `load_hessian(layer, hf_name)` and REPLACED by its packed layer.  Returns the per-layer metrics."""
    metrics = {}
    with torch.inference_mode():
        for name, module in list(full_model.named_modules()):
            match = re.fullmatch(_PROJ, name)
            if match is None or not isinstance(module, nn.Linear):
                continue
            layer, hf_name = int(match.group(1)), match.group(3) or match.group(4)
            H = load_hessian(layer, hf_name).to(module.weight.device)
            W = module.weight.detach().float()
            packed = quantize_layer(permute, H, W, shift_register_size, num_banks, batch_size,
                                    None if module.bias is None else module.bias.detach().float())
            metrics[name] = tuple(float(v) for v in evaluate_layer(H, W, packed.reconstruct()))
            if report:
                frob, proxy, proxy_diag, proxy_sum = metrics[name]
                report(f"{layer=}, {hf_name=}, frob={frob:g}, proxy={proxy:g}, proxy_diag={proxy_diag:g}, proxy_sum={proxy_sum:g}")
            swap_module(full_model, name, packed)
    return metrics


def swap_module(model: nn.Module, name: str, new: nn.Module) -> None:
    parent_name, _, leaf = name.rpartition(".")
    setattr(model.get_submodule(parent_name) if parent_name else model, leaf, new)


# ---- packed checkpoints -----------------------------------------------------------------------------------
def packed_checkpoint(model: nn.Module) -> dict:
    """state_dict plus the shapes needed to rebuild the packed layers in a freshly constructed model."""
    layers = {name: (mod.out_features, mod.in_features, mod.L, mod.num_banks, mod.bias is not None)
              for name, mod in model.named_modules() if isinstance(mod, FactorizedRPTCLinear)}
    return {"format": "rptc-factorized-v1", "layers": layers, "state": model.state_dict()}


def save_packed_safetensors(model: nn.Module, path) -> None:
    """The packed checkpoint as one safetensors file: the state dict's tensors, with the layer shapes that
    `load_packed_checkpoint` needs as JSON in the file's metadata."""
    import json

    from safetensors.torch import save_file
    ckpt = packed_checkpoint(model)
    tensors = {k: v.detach().cpu().contiguous() for k, v in ckpt["state"].items()}
    save_file(tensors, str(path), metadata={"format": ckpt["format"], "layers": json.dumps(ckpt["layers"])})


def load_packed_safetensors(model: nn.Module, path, device="cuda") -> nn.Module:
    """Reads a file written by `save_packed_safetensors` into `model` (built from its config, weights irrelevant)."""
    import json

    from safetensors import safe_open
    state = {}
    with safe_open(str(path), framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        for k in f.keys():
            state[k] = f.get_tensor(k)
    if meta.get("format") != "rptc-factorized-v1":
        raise ValueError("not a packed RPTC checkpoint")
    layers = {name: tuple(v) for name, v in json.loads(meta["layers"]).items()}
    return load_packed_checkpoint(model, {"format": meta["format"], "layers": layers, "state": state}, device=device)


def load_packed_checkpoint(model: nn.Module, ckpt: dict, device="cuda") -> nn.Module:
    """Swaps empty packed layers into `model` (built from its config, weights irrelevant) and loads the state."""
    if ckpt.get("format") != "rptc-factorized-v1":
        raise ValueError("not a packed RPTC checkpoint")
    for name, (m, n, L, banks, has_bias) in ckpt["layers"].items():
        swap_module(model, name, FactorizedRPTCLinear(m, n, L, banks, has_bias, device=device))
    model.load_state_dict(ckpt["state"])
    return model
