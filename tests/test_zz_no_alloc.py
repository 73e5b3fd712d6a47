"""GPU test of rptc_gemv_f16_static, the fused matvec for hosts that cannot allocate device memory
where they call the library (its fp32 accumulator is a fixed array inside the library).

Called through the C ABI and compared with the ordinary pair rptc_gemv + rptc_gemv_finish on the
same inputs, twice in a row (the second call finds the first call's leftovers in the shared
array).  Both paths add partial sums with atomics, so they may differ in the last bits: the
tolerance is the one the fused-matvec tests use (gpu_util.py: 1.5e-4 * ||w_row|| * ||x|| for the batch-1
kernel, 2e-5 for the tensor-core kernel that serves batch 2, plus the fp16 rounding of the result), taken
against the fp64 product of the decoded weights.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from gpu_util import GEMV_FP32_TOL, GEMV_HFMA2_TOL

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
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _static(L, codes, lut, x, y_new, m, n, fmt)
        torch.cuda.synchronize()
        if call == 1:      # the first call may load the library's kernels; from then on the device's free memory must not move
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point allocated device memory"
        y_old = ops.gemv(codes, lut, x, m, n, fmt)
        torch.cuda.synchronize()
        exact = x.double() @ dense.t()
        rel = torch.full((batch, 1), GEMV_FP32_TOL, dtype=torch.float64, device="cuda")
        if batch % 2:
            rel[-1] = GEMV_HFMA2_TOL                          # an odd batch ends in a batch-1 launch
        tol = rel * x.double().norm(dim=1)[:, None] * wnorm[None, :] + 2.0**-11 * exact.abs() + 1e-4
        assert bool(((y_new.double() - exact).abs() <= tol).all()), f"call {call}: static path off"
        assert bool(((y_new.double() - y_old.double()).abs() <= 2 * tol).all()), f"call {call}: paths disagree"
    ops.device_status()


def test_static_accumulator_rejects_sizes_beyond_its_array():
    from rptc_b200 import Format, lib
    fmt = Format()
    st = lib().rptc_gemv_f16_static(1 << 8, 1 << 8, None, 1 << 8, 64, 1 << 8, 1 << 20, 262144 // 8 + 32, 64, 8, 0,
                                    ctypes.byref(fmt), None)
    assert st == -7                                          # RPTC_ERR_TOO_LARGE, before anything is launched


def test_static_accumulator_at_exactly_its_limit():
    """batch * m == 262144 floats fills the fixed array to the last element: accepted, and the last row is right."""
    from rptc_b200 import Format, lib, ops
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(3)
    m, n, batch = 32768, 256, 8
    fmt = Format()
    codes = torch.randint(-2**31, 2**31 - 1, (m // 32, n // 64, 32, 4), dtype=torch.int32, device="cuda", generator=g)
    lut = torch.randn(512, dtype=torch.float16, device="cuda", generator=g)
    x = torch.randn((batch, n), dtype=torch.float16, device="cuda", generator=g)
    y = torch.zeros((batch, m), dtype=torch.float16, device="cuda")
    _static(L, codes, lut, x, y, m, n, fmt)
    torch.cuda.synchronize()
    dense = ops.decompress(codes, lut, m, n, fmt).double()
    exact = x.double() @ dense.t()
    tol = GEMV_FP32_TOL * x.double().norm(dim=1)[:, None] * dense.norm(dim=1)[None, :] + 2.0**-11 * exact.abs() + 1e-4
    assert bool(((y.double() - exact).abs() <= tol).all())
    ops.device_status()


def test_a_rejected_call_leaves_the_stream_alone():
    """A refused call (bad format) must not clear the shared array behind a valid call's back: run a valid call, then a
    refused one, then finish nothing further -- the valid call's result stands, and the refused call returned its
    error without queueing work (checked by the result being complete before any further synchronisation point)."""
    from rptc_b200 import Format, lib, ops
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(4)
    m, n = 1024, 2048
    fmt = Format()
    codes = torch.randint(-2**31, 2**31 - 1, (m // 32, n // 64, 32, 4), dtype=torch.int32, device="cuda", generator=g)
    lut = torch.randn(512, dtype=torch.float16, device="cuda", generator=g)
    x = torch.randn((1, n), dtype=torch.float16, device="cuda", generator=g)
    y = torch.zeros((1, m), dtype=torch.float16, device="cuda")
    _static(L, codes, lut, x, y, m, n, fmt)
    bad = Format(code=1, K=4)
    st = L.rptc_gemv_f16_static(codes.data_ptr(), lut.data_ptr(), None, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
                                m, n, 1, 0, ctypes.byref(bad), torch.cuda.current_stream().cuda_stream)
    assert st == -4
    torch.cuda.synchronize()
    want = ops.gemv(codes, lut, x, m, n, fmt)
    assert (y.float() - want.float()).abs().max().item() <= 2.0**-10 * want.float().abs().max().item() + 1e-3
