"""GPU parity: the randomized Hadamard kernel against the oracle's float64 transform.
Tolerance: the kernel works in fp32 and rounds the result to fp16 once -> |err| <= 2^-10 |y| + 1e-3."""
import numpy as np
import pytest
import torch

import rptc_oracle as o
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,block", [(4096, 4096), (8192, 4096), (11008, 256), (28672, 4096), (1024, 512), (512, 64), (256, 8)])
@pytest.mark.parametrize("rows", [1, 5])
@pytest.mark.parametrize("transpose", [False, True])
def test_hadamard_fp16_in(n, block, rows, transpose):
    from rptc_b200 import ops
    rng = np.random.default_rng(n + block + rows)
    x = rng.standard_normal((rows, n)).astype(np.float16)
    s = o.signs_from_seed(n, n).astype(np.float16)
    ref = o.rht(x.astype(np.float64), s.astype(np.float64), block, transpose=transpose) * 0.5
    y = ops.hadamard(to_dev(x), to_dev(s), block, transpose=transpose, scale=0.5)
    err = np.abs(y.float().cpu().numpy() - ref)
    assert (err <= 2.0**-10 * np.abs(ref) + 1e-3).all()


def test_hadamard_fp32_in_clear_and_inverse():
    from rptc_b200 import ops
    rng = np.random.default_rng(3)
    n, block = 11008, o.hadamard_block(11008)
    x = rng.standard_normal((2, n)).astype(np.float32)
    s = o.signs_from_seed(1, n).astype(np.float16)
    xd = to_dev(x)
    y = ops.hadamard(xd, to_dev(s), block, transpose=False, clear_in=True)
    assert bool((xd == 0).all())
    ref = o.rht(x, s.astype(np.float64), block)
    assert (np.abs(y.float().cpu().numpy() - ref) <= 2.0**-10 * np.abs(ref) + 1e-3).all()
    back = ops.hadamard(y, to_dev(s), block, transpose=True)
    assert np.allclose(back.float().cpu().numpy(), x, atol=2e-2)


def _glue_reference(acc, s_out, scale, h, w_norm, eps, s_in, transform_in):
    """fp64 statement of the decoder-block glue: residual update, RMSNorm, next layer's input transform."""
    n = acc.shape[-1]
    block = min(n, 4096)                                     # 8192-wide rows are two blocks of 4096
    h_new = h.astype(np.float64) + o.rht(acc, s_out, block, transpose=True) * scale
    h16 = h_new.astype(np.float16).astype(np.float64)
    xn = h16 / np.sqrt((h16 ** 2).mean(-1, keepdims=True) + eps) * w_norm.astype(np.float64)
    xn = xn.astype(np.float16).astype(np.float64)
    return h_new, (o.rht(xn, s_in, block) if transform_in else xn)


@pytest.mark.parametrize("n", [256, 1024, 4096, 8192])
@pytest.mark.parametrize("transform_in", [True, False])
def test_finish_norm_hadamard(n, transform_in):
    from rptc_b200 import ops
    rng = np.random.default_rng(n + transform_in)
    rows = 2
    acc = rng.standard_normal((rows, n)).astype(np.float32)
    h = rng.standard_normal((rows, n)).astype(np.float16)
    w_norm = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    s_out, s_in = o.signs_from_seed(5, n), o.signs_from_seed(6, n)
    ref_h, ref_out = _glue_reference(acc, s_out, 0.37, h, w_norm, 1e-5, s_in, transform_in)
    d_acc, d_h, out = to_dev(acc), to_dev(h), torch.empty(rows, n, dtype=torch.float16, device="cuda")
    ops.finish_norm_hadamard(d_acc, to_dev(s_out.astype(np.float16)), 0.37, d_h, to_dev(w_norm), 1e-5,
                             to_dev(s_in.astype(np.float16)), transform_in, out)
    torch.cuda.synchronize()
    assert not d_acc.any()                                   # accumulator handed back cleared
    np.testing.assert_allclose(d_h.float().cpu().numpy(), ref_h, atol=4e-3, rtol=2e-3)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref_out, atol=1e-2, rtol=5e-3)


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("m", [4096, 22016])
@pytest.mark.parametrize("with_acc", [True, False])
def test_gemv_computing_its_own_input_matches_glue_then_gemv(batch, m, with_acc):
    """rptc_gemv_glued against rptc_finish_norm_hadamard followed by rptc_gemv, several calls in a row."""
    from gpu_util import rand_lut, rand_words
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(batch * 7 + m + with_acc)
    n = 4096
    fmt = Format(o.CODE_B, 2, 16, 8, o.LAYOUT_TILED)
    codes = to_dev(o.from_rowmajor(rand_words(rng, m, n, 2), o.LAYOUT_TILED))
    lut = to_dev(rand_lut(rng, o.CODE_B, S=8))
    w_norm = to_dev((1 + 0.1 * rng.standard_normal(n)).astype(np.float16))
    s_out, s_in = to_dev(o.signs_from_seed(7, n).astype(np.float16)), to_dev(o.signs_from_seed(8, n).astype(np.float16))
    dirty = torch.ones(1024, dtype=torch.float32, device="cuda")
    for rep in range(3):
        prev = to_dev(rng.standard_normal((batch, n)).astype(np.float32)) if with_acc else None
        h0 = to_dev(rng.standard_normal((batch, n)).astype(np.float16))
        h_a, x_a = h0.clone(), torch.empty_like(h0)
        acc_a = torch.zeros(batch, m, dtype=torch.float32, device="cuda")
        ops.finish_norm_hadamard(prev.clone() if with_acc else None, s_out, 0.3, h_a, w_norm, 1e-5, s_in, True, x_a)
        ops.gemv_acc(codes, lut, x_a, acc_a, m, n, fmt)
        h_b, acc_b = torch.full_like(h0, float("nan")), torch.zeros_like(acc_a)
        keep = prev.clone() if with_acc else None
        ops.gemv_norm_input(codes, lut, acc_b, m, n, fmt, batch, prev, s_out, 0.3, h0, h_b, w_norm, 1e-5, s_in, clear=dirty)
        torch.cuda.synchronize()
        ops.device_status()
        assert torch.equal(h_b, h_a)                           # same arithmetic, one writer
        assert not dirty.any()
        dirty.fill_(1.0)
        if with_acc:
            assert torch.equal(prev, keep)                     # read by every CTA, cleared by none
        # identical activations; the partial sums meet in a different order
        scale = acc_a.abs().max().item()
        assert (acc_b - acc_a).abs().max().item() <= 5e-4 * scale


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("m,n,block,code,K,S", [(4096, 11008, 256, o.CODE_B, 2, 8), (4096, 1792, 256, o.CODE_B, 2, 8),
                                                (64, 512, 128, o.CODE_B, 2, 8), (1056, 2048, 64, o.CODE_B, 2, 8),
                                                (1056, 2048, 256, o.CODE_A, 4, 0), (352, 1024, 256, o.CODE_C, 2, 9),
                                                (352, 1024, 32, o.CODE_C, 4, 9), (128, 768, 256, o.CODE_A, 2, 0)])
def test_down_projection_making_its_own_swiglu_input(batch, m, n, block, code, K, S):
    """rptc_gemv_swiglu against rptc_swiglu_hadamard followed by rptc_gemv, several calls in a row."""
    from gpu_util import rand_lut, rand_words
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(batch * 11 + m + n + K)
    fmt = Format(code, K, 16, S, o.LAYOUT_TILED)
    codes = to_dev(o.from_rowmajor(rand_words(rng, m, n, K), o.LAYOUT_TILED))
    lut = to_dev(rand_lut(rng, code, 16, S))
    s_out, s_in = to_dev(o.signs_from_seed(3, 2 * n).astype(np.float16)), to_dev(o.signs_from_seed(4, n).astype(np.float16))
    dirty = torch.ones(2048, dtype=torch.float32, device="cuda")
    for rep in range(3):
        prev = to_dev(rng.standard_normal((batch, 2 * n)).astype(np.float32))
        keep = prev.clone()
        x_a = torch.empty((batch, n), dtype=torch.float16, device="cuda")
        ops.swiglu_hadamard(prev.clone(), x_a, s_out, s_in, n, block, 0.7, 1.0, clear=True)
        acc_a = torch.zeros(batch, m, dtype=torch.float32, device="cuda")
        ops.gemv_acc(codes, lut, x_a, acc_a, m, n, fmt)
        acc_b = torch.zeros_like(acc_a)
        ops.gemv_swiglu_input(codes, lut, acc_b, m, n, fmt, batch, prev, s_out, 0.7, s_in, block, clear=dirty)
        torch.cuda.synchronize()
        ops.device_status()
        assert torch.equal(prev, keep) and not dirty.any()
        dirty.fill_(1.0)
        # identical activations; the products are summed in fp16 groups here and, at batch 2, in fp32 by the
        # tensor-core kernel on the other side
        scale = acc_a.abs().max().item()
        assert (acc_b - acc_a).abs().max().item() <= (5e-4 if batch == 1 else 2e-3) * scale


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("with_acc", [True, False])
def test_gemv_computing_its_own_input_from_8192_wide_rows(batch, with_acc):
    """rptc_gemv_glued with n = 8192 (two 4096-point blocks per row) against the separate glue kernel + rptc_gemv."""
    from gpu_util import rand_lut, rand_words
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(batch * 5 + with_acc)
    m, n = 1280, 8192
    fmt = Format(o.CODE_B, 2, 16, 8, o.LAYOUT_TILED)
    codes = to_dev(o.from_rowmajor(rand_words(rng, m, n, 2), o.LAYOUT_TILED))
    lut = to_dev(rand_lut(rng, o.CODE_B, S=8))
    w_norm = to_dev((1 + 0.1 * rng.standard_normal(n)).astype(np.float16))
    s_out, s_in = to_dev(o.signs_from_seed(7, n).astype(np.float16)), to_dev(o.signs_from_seed(8, n).astype(np.float16))
    for rep in range(2):
        prev = to_dev(rng.standard_normal((batch, n)).astype(np.float32)) if with_acc else None
        h0 = to_dev(rng.standard_normal((batch, n)).astype(np.float16))
        h_a, x_a = h0.clone(), torch.empty_like(h0)
        acc_a = torch.zeros(batch, m, dtype=torch.float32, device="cuda")
        ops.finish_norm_hadamard(prev.clone() if with_acc else None, s_out, 0.3, h_a, w_norm, 1e-5, s_in, True, x_a)
        ops.gemv_acc(codes, lut, x_a, acc_a, m, n, fmt)
        h_b, acc_b = torch.full_like(h0, float("nan")), torch.zeros_like(acc_a)
        ops.gemv_norm_input(codes, lut, acc_b, m, n, fmt, batch, prev, s_out, 0.3, h0, h_b, w_norm, 1e-5, s_in)
        torch.cuda.synchronize()
        ops.device_status()
        assert torch.equal(h_b, h_a)
        scale = acc_a.abs().max().item()
        # the sum of squares is accumulated in a different order (16 values a thread instead of 8), so activations can
        # differ by an fp16 ulp
        assert (acc_b - acc_a).abs().max().item() <= 2e-3 * scale
