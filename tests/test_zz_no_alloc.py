"""GPU test of rptc_gemv_f16_static, the fused matvec for hosts that cannot allocate device memory
where they call the library (its fp32 accumulator is a fixed array inside the library).

Called through the C ABI and compared with the ordinary pair rptc_gemv + rptc_gemv_finish on the
same inputs, twice in a row (the second call finds the first call's leftovers in the shared
array).  Both paths add partial sums with atomics, so they may differ in the last bits: the
tolerance is the one the fused-matvec tests use, 2e-3 * ||w_row|| * ||x|| + 1e-3 |y| + 1e-3, taken
against the fp64 product of the decoded weights.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _static(lib, codes, lut, x, y, m, n, fmt):
    st = lib.rptc_gemv_f16_static(codes.data_ptr(), lut.data_ptr(), None, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
                                  m, n, x.shape[0], 0, ctypes.byref(fmt), torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.rptc_strerror(st)


@pytest.mark.parametrize("batch", [1, 3])
def test_static_accumulator_matches_the_scratch_path_twice(batch):
    from rptc_b200 import Format, lib, ops
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(17 + batch)
    m, n = 4096, 4096
    fmt = Format()                                           # HASH, K=2, TILED
    codes = torch.randint(-2**31, 2**31 - 1, (m // 32, n // 64, 32, 4), dtype=torch.int32, device="cuda", generator=g)
    lut = torch.randn(512, dtype=torch.float16, device="cuda", generator=g)
    dense = ops.decompress(codes, lut, m, n, fmt).double()
    wnorm = dense.norm(dim=1)
    for call in range(2):
        x = torch.randn((batch, n), dtype=torch.float16, device="cuda", generator=g)
        y_new = torch.full((batch, m), 9.0, dtype=torch.float16, device="cuda")
        _static(L, codes, lut, x, y_new, m, n, fmt)
        y_old = ops.gemv(codes, lut, x, m, n, fmt)
        torch.cuda.synchronize()
        exact = x.double() @ dense.t()
        tol = 2e-3 * x.double().norm(dim=1)[:, None] * wnorm[None, :] + 1e-3 * exact.abs() + 1e-3
        assert bool(((y_new.double() - exact).abs() <= tol).all()), f"call {call}: static path off"
        assert bool(((y_new.double() - y_old.double()).abs() <= 2 * tol).all()), f"call {call}: paths disagree"
    ops.device_status()


def test_static_accumulator_rejects_sizes_beyond_its_array():
    from rptc_b200 import Format, lib
    fmt = Format()
    st = lib().rptc_gemv_f16_static(1 << 8, 1 << 8, None, 1 << 8, 64, 1 << 8, 1 << 20, 262144 // 8 + 32, 64, 8, 0,
                                    ctypes.byref(fmt), None)
    assert st == -7                                          # RPTC_ERR_TOO_LARGE, before anything is launched
