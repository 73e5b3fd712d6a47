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
