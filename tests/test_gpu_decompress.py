"""GPU parity: rptc_decompress (through the C ABI) is bit-exact against the CPU oracle."""
import numpy as np
import pytest
import torch

import rptc_oracle as o
from gpu_util import bits, lut_for_oracle, rand_lut, rand_words, to_dev

pytestmark = pytest.mark.gpu

CASES = [  # code, K, L, S
    (o.CODE_A, 2, 16, 0), (o.CODE_A, 3, 16, 0), (o.CODE_A, 4, 16, 0), (o.CODE_A, 2, 14, 0),
    (o.CODE_B, 2, 16, 8), (o.CODE_B, 2, 16, 6), (o.CODE_C, 2, 16, 9), (o.CODE_C, 4, 16, 9), (o.CODE_C, 2, 12, 7),
]


@pytest.mark.parametrize("code,K,L,S", CASES)
@pytest.mark.parametrize("layout", [o.LAYOUT_ROWMAJOR, o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR, o.LAYOUT_TILED])
@pytest.mark.parametrize("m,n", [(32, 2048), (96, 4096), (64, 6144)])
def test_decompress_bit_exact(code, K, L, S, layout, m, n):
    from rptc_b200 import Format, ops
    if layout == o.LAYOUT_CHUNKED and (n * K // 128) % 32:
        pytest.skip("chunked layout needs a multiple of 32 units per row")
    rng = np.random.default_rng(hash((code, K, L, S, layout, m, n)) % 2**32)
    w = rand_words(rng, m, n, K)
    lut = rand_lut(rng, code, L, S)
    ref = o.decode(w, lut_for_oracle(lut, code, S), n, code=code, K=K, L=L, S=S)
    fmt = Format(code, K, L, S, layout)
    got = ops.decompress(to_dev(o.from_rowmajor(w, layout)), to_dev(lut), m, n, fmt)
    torch.cuda.synchronize()
    assert np.array_equal(bits(got), bits(ref))
    ops.device_status()


@pytest.mark.parametrize("layout", [o.LAYOUT_ROWMAJOR, o.LAYOUT_UNITMAJOR, o.LAYOUT_TILED])
def test_decompress_ragged_width_and_carry(layout):
    # n = 11008 (172 units: not a multiple of 32) with a left-shard halo, and a padded output pitch
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(21)
    m, n = 64, 11008
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, o.CODE_B, S=8)
    ci = rng.integers(0, 2**32, m, dtype=np.uint64).astype(np.uint32)
    ref = o.decode(w, lut, n, code=o.CODE_B, S=8, carry_in=ci)
    out = torch.full((m, n + 64), 7.0, dtype=torch.float16, device="cuda")
    ops.decompress(to_dev(o.from_rowmajor(w, layout)), to_dev(lut), m, n, Format(o.CODE_B, 2, 16, 8, layout),
                   out=out[:, :n], carry_in=to_dev(ci))
    torch.cuda.synchronize()
    assert np.array_equal(bits(out[:, :n].contiguous()), bits(ref))
    assert bool((out[:, n:] == 7.0).all()), "columns beyond n must not be written"


@pytest.mark.parametrize("quirk,code,S", [(o.QUIRK_K1_LANE0_SEED, o.CODE_A, 0), (o.QUIRK_K2_LANE0_CARRY, o.CODE_B, 8)])
@pytest.mark.parametrize("layout", [o.LAYOUT_ROWMAJOR, o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR, o.LAYOUT_TILED])
def test_decompress_reference_quirks(quirk, code, S, layout):
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(31 + quirk)
    m, n = 64, 6144
    w = rand_words(rng, m, n, 2)
    lut = rand_lut(rng, code, 16, S)
    ref = o.decode(w, lut, n, code=code, S=S, quirk=quirk)
    got = ops.decompress(to_dev(o.from_rowmajor(w, layout)), to_dev(lut), m, n, Format(code, 2, 16, S, layout, quirk))
    torch.cuda.synchronize()
    assert np.array_equal(bits(got), bits(ref))


@pytest.mark.parametrize("m,n,K", [(4096, 4096, 2), (4096, 11008, 3), (11008, 4096, 4)])
def test_decompress_full_size_against_c_oracle(m, n, K):
    # BASELINE-size matrices: the multi-threaded C oracle is fast enough to check every element
    import c_oracle
    from rptc_b200 import Format, ops
    rng = np.random.default_rng(m + n + K)
    rm = rand_words(rng, m, n, K)
    lut = rand_lut(rng, o.CODE_A)
    ref = c_oracle.decompress(rm, lut, m, n, code=0, K=K, layout=o.LAYOUT_ROWMAJOR)
    got = ops.decompress(to_dev(o.from_rowmajor(rm, o.LAYOUT_TILED)), to_dev(lut), m, n, Format(o.CODE_A, K, 16, 0, o.LAYOUT_TILED))
    torch.cuda.synchronize()
    assert np.array_equal(bits(got), bits(ref))


def test_repack_round_trip_and_oracle():
    from rptc_b200 import ops
    rng = np.random.default_rng(41)
    m, nu = 96, 64
    w = rand_words(rng, m, nu * 64, 2)
    d = to_dev(w)
    for dst in (o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR, o.LAYOUT_TILED):
        r = ops.repack(d, o.LAYOUT_ROWMAJOR, dst, m, nu)
        assert np.array_equal(r.cpu().numpy().view(np.uint32), o.from_rowmajor(w, dst))
        back = ops.repack(r, dst, o.LAYOUT_ROWMAJOR, m, nu)
        assert torch.equal(back, d)
    c = ops.repack(d, o.LAYOUT_ROWMAJOR, o.LAYOUT_CHUNKED, m, nu)
    u = ops.repack(c, o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR, m, nu)
    assert np.array_equal(u.cpu().numpy().view(np.uint32), o.from_rowmajor(w, o.LAYOUT_UNITMAJOR))
    t = ops.repack(u, o.LAYOUT_UNITMAJOR, o.LAYOUT_TILED, m, nu)
    assert np.array_equal(t.cpu().numpy().view(np.uint32), o.from_rowmajor(w, o.LAYOUT_TILED))


def test_bad_arguments_raise():
    from rptc_b200 import Format, RPTCError, ops
    codes = torch.zeros((32, 8), dtype=torch.int32, device="cuda")
    lut = torch.zeros(512, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.decompress(codes, lut[:100], 32, 128, Format(o.CODE_B, 2, 16, 8, o.LAYOUT_ROWMAJOR))
    with pytest.raises(RPTCError):
        ops.decompress(codes[:24].contiguous(), lut, 24, 128, Format(o.CODE_B, 2, 16, 8, o.LAYOUT_ROWMAJOR))
