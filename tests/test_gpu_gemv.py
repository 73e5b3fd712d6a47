"""GPU parity: the fused dequant-GEMV against the CPU oracle (fp64 product of bit-exact weights).

Tolerance (derived in gpu_util.py from the kernels' arithmetic).  Batch 1 multiplies in fp16 pairs and adds eight
products per fp16 accumulator before widening to fp32: |y - exact| <= 1.5e-4 ||w_row|| ||x|| + 2^-11 |exact|, which is
0.6 absolute at n = 4096 with N(0,1) data -- below the ~1 that ONE mis-decoded weight moves an output by (the
reference's fully fp16-accumulated product, inference.cu:263,270-276, is about 200 times looser).  Batch 2-8 runs on
mma.sync with fp32 accumulation: 2e-5 ||w_row|| ||x||.  Wrong weights are hunted exactly, column by column, in
test_gpu_probe.py; this file checks the arithmetic on random inputs.
"""
import numpy as np
import pytest
import torch

import rptc_oracle as o
from gpu_util import GEMV_FP32_TOL, GEMV_HFMA2_TOL, bits, check_product, lut_for_oracle, rand_lut, rand_words, to_dev

pytestmark = pytest.mark.gpu


def _check(y, w16, x16, rel=None, what=""):
    """rel defaults to the bound of the kernel that serves this batch size (1: HFMA2, 2-8: mma.sync)."""
    if rel is None:
        rel = GEMV_HFMA2_TOL if x16.shape[0] in (1, 3, 5, 7) else GEMV_FP32_TOL      # odd batches end in a batch-1 launch
    exact = o.matvec_exact(w16, x16)
    check_product(y, exact, np.linalg.norm(w16.astype(np.float64), axis=1), np.linalg.norm(x16.astype(np.float64), axis=1), rel, what)


CASES = [(o.CODE_B, 2, 16, 8), (o.CODE_B, 2, 16, 6), (o.CODE_A, 2, 16, 0), (o.CODE_A, 4, 16, 0), (o.CODE_A, 2, 14, 0),
         (o.CODE_C, 2, 16, 9), (o.CODE_C, 4, 16, 9)]


@pytest.mark.parametrize("code,K,L,S", CASES)
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("m,n", [(64, 2048), (4096, 4096), (352, 11008)])
def test_gemv_native_layout(code, K, L, S, batch, m, n):
    from rptc_b200 import Format, ops
    if code != o.CODE_B and batch not in (1, 4) :
        pytest.skip("batch sweep runs on the headline code only")
    rng = np.random.default_rng(hash((code, K, L, S, batch, m, n)) % 2**32)
    w = rand_words(rng, m, n, K)
    lut = rand_lut(rng, code, L, S)
    x = rng.standard_normal((batch, n)).astype(np.float16)
    w16 = o.decode(w, lut_for_oracle(lut, code, S), n, code=code, K=K, L=L, S=S)
    y = ops.gemv(to_dev(o.from_rowmajor(w, o.LAYOUT_TILED)), to_dev(lut), to_dev(x), m, n,
                 Format(code, K, L, S, o.LAYOUT_TILED))
    torch.cuda.synchronize()
    ops.device_status()
    _check(y.float().cpu().numpy(), w16, x)


@pytest.mark.parametrize("layout", [o.LAYOUT_ROWMAJOR, o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR])
def test_gemv_legacy_layouts(layout):
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(51 + layout)
    m, n = 128, 4096
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    x = rng.standard_normal((1, n)).astype(np.float16)
    w16 = o.decode(w, lut, n, code=o.CODE_B, S=8)
    y = ops.gemv(to_dev(o.from_rowmajor(w, layout)), to_dev(lut), to_dev(x), m, n, Format(o.CODE_B, 2, 16, 8, layout))
    _check(y.float().cpu().numpy(), w16, x, GEMV_HFMA2_TOL)      # the general kernel is an HFMA2 kernel


def test_gemv_carry_in_and_column_sharding():
    # a row-parallel (column-sharded) layer: shard s decodes units [s*U/2, (s+1)*U/2) and needs the 16 bits
    # before its first unit; the partial products add up to the unsharded result
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(61)
    m, n = 256, 8192
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    x = rng.standard_normal((2, n)).astype(np.float16)
    w16 = o.decode(w, lut, n, code=o.CODE_B, S=8)
    nw = w.shape[1]
    left, right = w[:, : nw // 2], w[:, nw // 2:]           # two column shards of the row-major stream
    acc = torch.zeros((2, m), dtype=torch.float32, device="cuda")
    fmt = Format(o.CODE_B, 2, 16, 8, o.LAYOUT_TILED)
    xd = to_dev(x)
    ops.gemv_acc(to_dev(o.from_rowmajor(left, o.LAYOUT_TILED)), to_dev(lut), xd[:, : n // 2], acc, m, n // 2, fmt)
    carry = np.ascontiguousarray(left[:, -1])               # last word of the left shard = the right shard's history
    ops.gemv_acc(to_dev(o.from_rowmajor(right, o.LAYOUT_TILED)), to_dev(lut), xd[:, n // 2:], acc, m, n // 2, fmt,
                 carry_in=to_dev(carry))
    torch.cuda.synchronize()
    _check(acc.cpu().numpy(), w16, x)


def test_gemv_finish_accumulate_and_clear():
    from rptc_b200 import ops
    acc = torch.arange(64, dtype=torch.float32, device="cuda").reshape(2, 32).contiguous()
    y = torch.ones((2, 32), dtype=torch.float16, device="cuda")
    ops.gemv_finish(acc, y, 32, scale=0.5, accumulate=True, clear=True)
    torch.cuda.synchronize()
    assert torch.equal(y.float().cpu(), 1 + 0.5 * torch.arange(64, dtype=torch.float32).reshape(2, 32))
    assert bool((acc == 0).all())


def test_gemv_all_ones_codebook_known_answer():
    # rptc_kernels/tests/test_decompress.py:11,38 — with an all-ones LUT every output equals sum(x)
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(71)
    m, n = 512, 8192
    w = rand_words(rng, m, n, 2)
    lut = np.ones(1 << 16, dtype=np.float16)
    x = rng.standard_normal((1, n)).astype(np.float16)
    y = ops.gemv(to_dev(o.from_rowmajor(w, o.LAYOUT_TILED)), to_dev(lut), to_dev(x), m, n,
                 Format(o.CODE_A, 2, 16, 0, o.LAYOUT_TILED))
    s = x.astype(np.float64).sum()
    assert np.allclose(y.float().cpu().numpy(), s, atol=2.0**-11 * abs(s) + 1.5e-4 * np.sqrt(n) * np.linalg.norm(x.astype(np.float64)))


@pytest.mark.parametrize("m,n", [(4096, 4096), (11008, 4096), (4096, 11008), (28672, 8192)])
def test_gemv_full_size_linearity(m, n):
    # BASELINE-size layers: checked through properties that need no CPU decode — linearity in x and
    # agreement with decompress-then-matmul on the GPU's own bit-exact decompress output
    from rptc_b200 import Format, ops
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    codes = torch.randint(-2**31, 2**31 - 1, (m // 32, n // 64, 32, 4), dtype=torch.int32, device="cuda", generator=g)
    lut = torch.randn(512, dtype=torch.float16, device="cuda", generator=g)
    x = torch.randn((2, n), dtype=torch.float16, device="cuda", generator=g)
    fmt = Format(o.CODE_B, 2, 16, 8, o.LAYOUT_TILED)
    y = ops.gemv(codes, lut, x, m, n, fmt).float()
    ysum = ops.gemv(codes, lut, (x[0] + x[1]).unsqueeze(0), m, n, fmt).float()      # the fp16 sum is the input of both sides
    dense = ops.decompress(codes, lut, m, n, fmt)
    ref = (x.double() @ dense.double().T)
    scale = dense.double().norm(dim=1)[None, :] * x.double().norm(dim=1)[:, None]
    err = (y.double() - ref).abs()
    tol = GEMV_FP32_TOL * scale + 2.0**-11 * ref.abs() + 1e-4                        # batch 2: the mma.sync kernel
    assert bool((err <= tol).all()), f"max err/tol {(err / tol).max().item():.3f}"
    # batch 1 (HFMA2 kernel) on the fp16 sum of the two rows, against the same product
    xs = (x[0] + x[1]).unsqueeze(0)
    ref_s = xs.double() @ dense.double().T
    err_s = (ysum.double() - ref_s).abs()
    tol_s = GEMV_HFMA2_TOL * dense.double().norm(dim=1)[None, :] * xs.double().norm() + 2.0**-11 * ref_s.abs() + 1e-4
    assert bool((err_s <= tol_s).all()), f"batch 1 max err/tol {(err_s / tol_s).max().item():.3f}"
