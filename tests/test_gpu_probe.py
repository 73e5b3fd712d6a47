"""GPU parity of the fused dequant-GEMV kernels by exact-column probes.

A random-input test with a norm-wise tolerance cannot see a handful of mis-decoded weights per row, and that is the
defect this path is prone to: the reference's own kernels have it twice (inference.cu:61-62 seeds lane 0 from the
wrong half-word, inference.cu:232 hands lane 0 its own word as carry: 6-7 wrong weights per 2048 columns).  The
history hand-over of the fused kernels (first unit of a warp's range, first unit of a run after a row-block change,
column-block starts, the shuffle between lanes of the tensor-core form, a column shard's first unit) is separate code
from the bit-exact decompress kernel, so it is probed here directly.

With an activation row that is a unit vector e_c every product is a weight times one or zero and every partial sum a
weight plus zeros: exact in fp16 and fp32 whatever the order of the additions.  The output row must then equal
column c of the decoded matrix BIT FOR BIT.  All n columns are probed (n / batch launches), so every boundary is hit.
The kernels that compute their activations inside the launch are probed the same way by choosing their inputs such
that the computed activation row is exactly 2^k * e_c.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

import rptc_oracle as o
from gpu_util import assert_same_bits, bits, lut_for_oracle, probe_columns, rand_lut, rand_words, to_dev

pytestmark = pytest.mark.gpu

BASELINE_SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (28672, 8192)]


def _random_layer(m, n, fmt, seed):
    from rptc_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    codes = torch.randint(-2**31, 2**31 - 1, ops.codes_shape(m, n, fmt.K, fmt.layout), dtype=torch.int32, device="cuda", generator=g)
    lut = torch.randn(fmt.lut_numel(), dtype=torch.float16, device="cuda", generator=g)
    return codes, lut


def _decoded(codes, lut, m, n, fmt, carry_in=None):
    """Bit-exact decode on the GPU (itself compared with the CPU oracle element for element in test_gpu_decompress.py,
    full BASELINE sizes included), spot-checked against the numpy oracle here as well."""
    from rptc_b200 import ops
    dense = ops.decompress(codes, lut, m, n, fmt, carry_in=carry_in)
    rows = min(m, 64)
    w = o.to_rowmajor(codes.cpu().numpy().view(np.uint32), fmt.layout)[:rows]
    ci = None if carry_in is None else carry_in.cpu().numpy().view(np.uint32)[:rows]
    ref = o.decode(w, lut_for_oracle(lut.cpu().numpy(), fmt.code, fmt.S), n, code=fmt.code, K=fmt.K, L=fmt.L, S=fmt.S, carry_in=ci)
    assert np.array_equal(bits(dense[:rows]), bits(ref))
    return dense


@pytest.mark.parametrize("m,n", BASELINE_SHAPES + [(352, 11008), (96, 2048)])
@pytest.mark.parametrize("batch", [1, 8])
def test_every_column_of_the_headline_code(m, n, batch):
    """HASH S=8 K=2, TILED: batch 1 is the HFMA2 pair kernel, batch 8 the mma.sync kernel (352 and 96 rows: an odd
    number of 32-row blocks, the last pair has no second block)."""
    from rptc_b200 import Format, ops
    fmt = Format()
    codes, lut = _random_layer(m, n, fmt, m * 3 + n + batch)
    dense = _decoded(codes, lut, m, n, fmt)
    Y = probe_columns(lambda x: ops.gemv(codes, lut, x, m, n, fmt), n, batch, m)
    torch.cuda.synchronize()
    ops.device_status()
    assert_same_bits(Y, dense.t(), f"{m}x{n} batch {batch}")


@pytest.mark.parametrize("batch", [2, 3, 4, 5, 7])
@pytest.mark.parametrize("m,n", [(4096, 4096), (352, 11008)])
def test_every_column_other_batches(m, n, batch):
    # 3, 5, 7 run as a short sequence of launches (4 + 1, 4 + 2 + 1, ...)
    from rptc_b200 import Format, ops
    fmt = Format()
    codes, lut = _random_layer(m, n, fmt, m + n + batch)
    dense = _decoded(codes, lut, m, n, fmt)
    Y = probe_columns(lambda x: ops.gemv(codes, lut, x, m, n, fmt), n, batch, m)
    assert_same_bits(Y, dense.t(), f"{m}x{n} batch {batch}")


@pytest.mark.parametrize("code,K,L,S", [(o.CODE_A, 2, 16, 0), (o.CODE_A, 4, 16, 0), (o.CODE_A, 2, 14, 0), (o.CODE_B, 2, 16, 6),
                                        (o.CODE_C, 2, 16, 9), (o.CODE_C, 4, 16, 9)])
@pytest.mark.parametrize("batch", [1, 8])
def test_every_column_other_codes(code, K, L, S, batch):
    from rptc_b200 import Format, ops
    m, n = 1024, 4096
    fmt = Format(code, K, L, S, o.LAYOUT_TILED)
    codes, lut = _random_layer(m, n, fmt, code * 100 + K * 10 + L + batch)
    dense = _decoded(codes, lut, m, n, fmt)
    Y = probe_columns(lambda x: ops.gemv(codes, lut, x, m, n, fmt), n, batch, m)
    ops.device_status()
    assert_same_bits(Y, dense.t(), f"code {code} K {K} L {L} batch {batch}")


@pytest.mark.parametrize("layout", [o.LAYOUT_ROWMAJOR, o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR])
@pytest.mark.parametrize("quirk", [o.QUIRK_NONE, o.QUIRK_K2_LANE0_CARRY, o.QUIRK_K1_LANE0_SEED])
def test_every_column_reference_layouts_and_quirks(layout, quirk):
    """The general kernel (the one behind the seven legacy entry points): the reference's three layouts, with and
    without the reference kernels' lane-0 deviations, against the numpy oracle itself."""
    from rptc_b200 import Format, ops
    m, n = 128, 6144 if layout != o.LAYOUT_CHUNKED else 4096
    rng = np.random.default_rng(7 + layout * 3 + quirk)
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    ref = torch.from_numpy(o.decode(w, lut, n, code=o.CODE_B, S=8, quirk=quirk)).cuda()
    fmt = Format(o.CODE_B, 2, 16, 8, layout, quirk)
    codes, lut_d = to_dev(o.from_rowmajor(w, layout)), to_dev(lut)
    Y = probe_columns(lambda x: ops.gemv(codes, lut_d, x, m, n, fmt), n, 1, m)
    assert_same_bits(Y, ref.t(), f"layout {layout} quirk {quirk}")


def test_every_column_legacy_activation_order():
    """decompress_matvec_*'s staging permutation (inference.cu:216-221,249): stream pair s multiplies the x pair
    k2_pair_source(n)[s], so a unit vector at column 2q+r returns stream column 2s+r with q[s] = q."""
    from rptc_b200 import XORDER_K2_LEGACY, Format, ops
    m, n = 128, 4096
    rng = np.random.default_rng(19)
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    ref = torch.from_numpy(o.decode(w, lut, n, code=o.CODE_B, S=8)).cuda()
    q = o.k2_pair_source(n)
    inv = np.empty_like(q)
    inv[q] = np.arange(len(q))
    stream_col = torch.from_numpy(2 * inv[np.arange(n) // 2] + np.arange(n) % 2).cuda()
    fmt = Format(o.CODE_B, 2, 16, 8, o.LAYOUT_CHUNKED)
    codes, lut_d = to_dev(o.from_rowmajor(w, o.LAYOUT_CHUNKED)), to_dev(lut)
    Y = probe_columns(lambda x: ops.gemv(codes, lut_d, x, m, n, fmt, x_order=XORDER_K2_LEGACY), n, 1, m)
    assert_same_bits(Y, ref.t()[stream_col], "legacy x order")


@pytest.mark.parametrize("batch", [1, 8])
@pytest.mark.parametrize("shards", [2, 8])
def test_every_column_of_a_column_shard(batch, shards):
    """Row-parallel tensor parallelism: shard s holds units [s U / shards, (s+1) U / shards) of every row and gets the
    16 stream bits in front of its first unit as carry_in.  Each shard's columns must equal the unsharded decode."""
    from rptc_b200 import Format, ops
    m, n = 256, 8192
    rng = np.random.default_rng(23 + shards)
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    ref = torch.from_numpy(o.decode(w, lut, n, code=o.CODE_B, S=8)).cuda()
    fmt = Format()
    lut_d = to_dev(lut)
    nw, ns = w.shape[1] // shards, n // shards
    for s in (0, 1, shards - 1):
        part = np.ascontiguousarray(w[:, s * nw:(s + 1) * nw])
        carry = None if s == 0 else to_dev(np.ascontiguousarray(w[:, s * nw - 1]))
        codes = to_dev(o.from_rowmajor(part, o.LAYOUT_TILED))
        Y = probe_columns(lambda x: ops.gemv(codes, lut_d, x, m, ns, fmt, carry_in=carry), ns, batch, m)
        assert_same_bits(Y, ref.t()[s * ns:(s + 1) * ns], f"shard {s} of {shards}")


def test_every_column_through_the_entry_point_without_scratch():
    from rptc_b200 import Format, lib, ops
    m, n = 4096, 4096
    fmt = Format()
    codes, lut = _random_layer(m, n, fmt, 29)
    dense = _decoded(codes, lut, m, n, fmt)
    L = lib()
    stream = torch.cuda.current_stream().cuda_stream

    def run(x):
        y = torch.empty((x.shape[0], m), dtype=torch.float16, device="cuda")
        st = L.rptc_gemv_f16_static(codes.data_ptr(), lut.data_ptr(), None, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
                                    m, n, x.shape[0], 0, ctypes.byref(fmt), stream)
        assert st == 0, L.rptc_strerror(st)
        return y

    for batch in (1, 8):
        Y = probe_columns(run, n, batch, m)
        assert_same_bits(Y, dense.t(), f"static entry point, batch {batch}")


# ---- kernels that make their activations inside the launch ----------------------------------------------------------
def _hadamard_column(block, c):
    """Column c of the natural-order (Sylvester) Hadamard matrix of size `block`: (-1)^popcount(i & c)."""
    i = np.arange(block)
    return 1.0 - 2.0 * (np.bitwise_count((i & c).astype(np.uint32)) & 1)


def _probe_cols(n, unit=64, extra=()):
    """Columns at every boundary the kernels treat specially, and a few in between."""
    cols = set(extra)
    for base in list(range(0, n, 2048)) + list(range(0, n, 4096)) + [n - 64, n - 256, n // 2]:
        for d in (-65, -64, -8, -2, -1, 0, 1, 2, 7, 8, 63, 64, 65, 255, 256, 257):
            if 0 <= base + d < n:
                cols.add(base + d)
    rng = np.random.default_rng(n)
    cols.update(int(c) for c in rng.integers(0, n, 24))
    return sorted(cols)


@pytest.mark.parametrize("rows", [1, 2])
@pytest.mark.parametrize("m,n", [(12288, 4096), (22016, 4096), (10240, 8192)])
@pytest.mark.parametrize("with_acc", [False, True])
def test_probe_matvec_that_computes_its_rmsnorm_input(m, n, rows, with_acc):
    """rptc_gemv_glued: x = H(s_in * rmsnorm(h') * w_norm) with h' = h_in + s_out * H(acc) * scale_out.  With
    h' = s_in * (column c of H) in every 4096-point block, w_norm = 1 and eps = 0 the row's mean square is exactly one
    and x = 64 * e_c per block: the accumulator must hold exactly 64 * (sum over blocks of W[:, c_b])."""
    from rptc_b200 import Format, ops
    fmt = Format()
    nb = n // 4096
    codes, lut = _random_layer(m, n, fmt, m + n + rows)
    dense = _decoded(codes, lut, m, n, fmt).float()
    g = torch.Generator(device="cuda").manual_seed(5)
    s_in = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    s_out = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    w_norm = torch.ones(n, dtype=torch.float16, device="cuda")
    scale_out = 0.5
    cols = _probe_cols(4096)
    cols += [cols[0]] * (-len(cols) % rows)
    acc = torch.zeros((rows, m), dtype=torch.float32, device="cuda")
    h_out = torch.zeros((rows, n), dtype=torch.float16, device="cuda")
    for i0 in range(0, len(cols), rows):
        want_h = np.zeros((rows, n))
        for r in range(rows):
            for b in range(nb):
                c = (cols[i0 + r] + 577 * b) % 4096           # a different column in every block
                want_h[r, 4096 * b:4096 * (b + 1)] = _hadamard_column(4096, c)
        want_h *= s_in.float().cpu().numpy()[None, :]
        if with_acc:
            # h_in = 0 and the previous layer's accumulator such that its output transform gives the pattern
            prev = o.rht(want_h, s_out.float().cpu().numpy(), 4096) / scale_out
            prev_acc = torch.from_numpy(prev.astype(np.float32)).cuda()
            h_in = torch.zeros((rows, n), dtype=torch.float16, device="cuda")
        else:
            prev_acc = None
            h_in = torch.from_numpy(want_h.astype(np.float16)).cuda()
        acc.zero_()
        ops.gemv_norm_input(codes, lut, acc, m, n, fmt, rows, prev_acc, s_out if with_acc else None, scale_out, h_in, h_out,
                            w_norm, 0.0, s_in)
        torch.cuda.synchronize()
        for r in range(rows):
            want = torch.zeros(m, dtype=torch.float32, device="cuda")
            for b in range(nb):
                want += dense[:, 4096 * b + (cols[i0 + r] + 577 * b) % 4096]
            got = acc[r] / 64.0
            assert torch.equal(got, want), f"columns {cols[i0 + r]}: {(got != want).sum().item()} rows differ"
        assert torch.equal(h_out.float().cpu(), torch.from_numpy(want_h).float()), "updated residual stream"
    ops.device_status()


@pytest.mark.parametrize("rows", [1, 2])
@pytest.mark.parametrize("m,n,block", [(4096, 11008, 256), (8192, 3584, 256), (4096, 1792, 64)])
def test_probe_down_projection_that_computes_its_swiglu_input(m, n, rows, block):
    """rptc_gemv_swiglu: x = H(s_in * fp16(silu(g) * u)) in blocks of `block` columns, (g | u) the output transform of
    the gate-up accumulator.  With g = 1 and u = +-u0 (u0 the fp16 number for which fp16(silu(1) * u0) is exactly 1) in
    one block and u = 0 elsewhere, x is exactly sqrt(block) * e_c (blocks of 4^k columns, so that the factor is a power of two)."""
    from rptc_b200 import Format, ops
    fmt = Format()
    codes, lut = _random_layer(m, n, fmt, m + n + rows + block)
    dense = _decoded(codes, lut, m, n, fmt).float()
    g = torch.Generator(device="cuda").manual_seed(6)
    s_in = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    s_out = (torch.randint(0, 2, (2 * n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    u0 = float(np.float16(1.0 / silu1))
    assert np.float16(silu1 * u0) == np.float16(1.0)
    scale_out = 0.25
    cols = _probe_cols(n)
    cols += [cols[0]] * (-len(cols) % rows)
    acc = torch.zeros((rows, m), dtype=torch.float32, device="cuda")
    si, so = s_in.float().cpu().numpy(), s_out.float().cpu().numpy()
    for i0 in range(0, len(cols), rows):
        target = np.zeros((rows, 2 * n))
        target[:, :n] = 1.0                                                    # gate
        for r in range(rows):
            c = cols[i0 + r]
            b0 = c - c % block
            target[r, n + b0:n + b0 + block] = u0 * si[b0:b0 + block] * _hadamard_column(block, c % block)
        prev = np.concatenate([o.rht(target[:, :n], so[:n], block), o.rht(target[:, n:], so[n:], block)], axis=1) / scale_out
        prev_acc = torch.from_numpy(prev.astype(np.float32)).cuda()
        acc.zero_()
        ops.gemv_swiglu_input(codes, lut, acc, m, n, fmt, rows, prev_acc, s_out, scale_out, s_in, block)
        torch.cuda.synchronize()
        for r in range(rows):
            got = acc[r] / math.sqrt(block)
            want = dense[:, cols[i0 + r]]
            assert torch.equal(got, want), f"column {cols[i0 + r]}: {(got != want).sum().item()} rows differ"
    ops.device_status()
