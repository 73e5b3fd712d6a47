"""GPU parity of the fused dequant-GEMM (tcgen05): against the product of the bit-exact decoded
weights (checked against the CPU oracle) with the same activations.

Tolerance: fp16 operands, fp32 accumulation in TMEM, one rounding to fp16 ->
|y - exact| <= 2^-10 |exact| + 5e-4 * ||w_row|| * ||x_t||."""
import numpy as np
import pytest
import torch

import rptc_oracle as o
from gpu_util import lut_for_oracle, rand_lut, rand_words, to_dev

pytestmark = pytest.mark.gpu


def _run(code, K, L, S, m, n, tokens, seed=0, check_oracle=True):
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(seed)
    w = rand_words(rng, m, n, K)
    lut = rand_lut(rng, code, L, S)
    fmt = Format(code, K, L, S, o.LAYOUT_TILED)
    codes = to_dev(o.from_rowmajor(w, o.LAYOUT_TILED))
    lut_d = to_dev(lut)
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((tokens, n), dtype=torch.float16, device="cuda", generator=g)
    y = ops.gemm(codes, lut_d, x, m, n, fmt)
    torch.cuda.synchronize()
    ops.device_status()
    dense = ops.decompress(codes, lut_d, m, n, fmt)
    if check_oracle:
        ref_w = o.decode(w[:32], lut_for_oracle(lut, code, S), n, code=code, K=K, L=L, S=S)
        assert np.array_equal(dense[:32].cpu().numpy().view(np.uint16), ref_w.view(np.uint16))
    exact = x.double() @ dense.double().t()
    scale = x.double().norm(dim=1)[:, None] * dense.double().norm(dim=1)[None, :]
    err = (y.double() - exact).abs()
    tol = 2.0**-10 * exact.abs() + 5e-4 * scale + 1e-4
    assert bool((err <= tol).all()), f"max err/tol {(err / tol).max().item():.3f}"


@pytest.mark.parametrize("m,n,tokens", [(128, 64, 256), (128, 512, 256), (256, 4096, 512), (128, 1024, 100), (384, 2048, 300)])
def test_gemm_hash_small(m, n, tokens):
    _run(o.CODE_B, 2, 16, 8, m, n, tokens, seed=m + n + tokens)


@pytest.mark.parametrize("code,K,L,S", [(o.CODE_A, 2, 16, 0), (o.CODE_A, 4, 16, 0), (o.CODE_A, 2, 14, 0), (o.CODE_B, 2, 16, 6),
                                        (o.CODE_C, 2, 16, 9), (o.CODE_C, 4, 16, 9)])
def test_gemm_all_codes(code, K, L, S):
    _run(code, K, L, S, 256, 2048, 384, seed=code * 7 + K)


@pytest.mark.parametrize("m,n,tokens", [(4096, 4096, 2048), (22016, 4096, 512), (4096, 11008, 512)])
def test_gemm_llama_shapes(m, n, tokens):
    _run(o.CODE_B, 2, 16, 8, m, n, tokens, seed=3, check_oracle=False)


def test_gemm_carry_in_column_shard():
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(5)
    m, n, tokens = 128, 2048, 256
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    fmt = Format(o.CODE_B, 2, 16, 8, o.LAYOUT_TILED)
    x = torch.randn((tokens, n), dtype=torch.float16, device="cuda")
    full = ops.gemm(to_dev(o.from_rowmajor(w, o.LAYOUT_TILED)), to_dev(lut), x, m, n, fmt).float()
    nw = w.shape[1]
    left, right = w[:, : nw // 2], w[:, nw // 2:]
    y1 = ops.gemm(to_dev(o.from_rowmajor(left, o.LAYOUT_TILED)), to_dev(lut), x[:, : n // 2].contiguous(), m, n // 2, fmt).float()
    y2 = ops.gemm(to_dev(o.from_rowmajor(right, o.LAYOUT_TILED)), to_dev(lut), x[:, n // 2:].contiguous(), m, n // 2, fmt,
                  carry_in=to_dev(np.ascontiguousarray(left[:, -1]))).float()
    assert (full - (y1 + y2)).abs().max() <= 2e-2 * full.abs().max()


def test_linear_prefill_path_matches_effective_weight():
    from rptc_b200.linear import RPTCLinear
    lin = RPTCLinear.random(4096, 1024, seed=9)
    x = torch.randn((300, 4096), dtype=torch.float16, device="cuda")
    y = lin(x).float()
    ref = x.float() @ lin.effective_weight().t()
    assert (y - ref).abs().max() <= 1e-2 * ref.abs().max()
