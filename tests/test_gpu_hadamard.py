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
    h_new = h.astype(np.float64) + o.rht(acc, s_out, n, transpose=True) * scale
    h16 = h_new.astype(np.float16).astype(np.float64)
    xn = h16 / np.sqrt((h16 ** 2).mean(-1, keepdims=True) + eps) * w_norm.astype(np.float64)
    xn = xn.astype(np.float16).astype(np.float64)
    return h_new, (o.rht(xn, s_in, n) if transform_in else xn)


@pytest.mark.parametrize("n", [256, 1024, 4096])
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
