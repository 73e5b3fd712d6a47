"""CPU tests: the numpy oracle against vectors produced by the reference's own Python code
(tests/golden/make_golden.py), against its own literal scan, and against the C oracle."""
import numpy as np
import pytest

import c_oracle
import rptc_oracle as o


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


@pytest.mark.parametrize("L", [16, 14])
def test_code_a_matches_reference_dequantize(golden, L):
    # rptc.py:74-85 run by the reference itself -> golden; the oracle decodes the packed stream
    alphabet, sym, ref = golden[f"a{L}_alphabet"], golden[f"a{L}_symbols"], golden[f"a{L}_decoded"]
    words = o.pack_symbols(sym, 2)
    got = o.decode(words, alphabet.astype(np.float16), sym.shape[1], code=o.CODE_A, K=2, L=L)
    assert np.array_equal(_bits(got), _bits(ref.astype(np.float16)))


def test_code_a_small_state_matches_reference_encode_decode(golden):
    # symbols chosen by the reference's Viterbi encoder (rptc.py:13-71), L = 8
    alphabet, sym, ref = golden["enc8_alphabet"], golden["enc8_symbols"], golden["enc8_decoded"]
    words = o.pack_symbols(sym, 2)
    got = o.decode(words, alphabet.astype(np.float16), sym.shape[1], code=o.CODE_A, K=2, L=8)
    assert np.array_equal(_bits(got), _bits(ref.astype(np.float16)))


def test_code_c_matches_reference_dequantize(golden):
    alphabet, sym, ref = golden["c_alphabet"], golden["c_symbols"], golden["c_decoded"]
    words = o.pack_symbols(sym, 4)
    n = sym.shape[1] * 2
    got = o.decode(words, alphabet.astype(np.float16), n, code=o.CODE_C, K=2, L=16, S=9)
    assert np.array_equal(_bits(got), _bits(ref.reshape(sym.shape[0], n).astype(np.float16)))
    assert np.array_equal(o.index_c(golden["c_index_states"], 16, 9), golden["c_index"].astype(np.uint32))


def test_code_c_small_state_matches_reference_encode_decode(golden):
    alphabet, sym, ref = golden["encc_alphabet"], golden["encc_symbols"], golden["encc_decoded"]
    words = o.pack_symbols(sym, 4)
    n = sym.shape[1] * 2
    got = o.decode(words, alphabet.astype(np.float16), n, code=o.CODE_C, K=2, L=8, S=5)
    assert np.array_equal(_bits(got), _bits(ref.reshape(sym.shape[0], n).astype(np.float16)))


@pytest.mark.parametrize("K", [2, 3, 4])
def test_code_a_windows_equal_literal_scan(K):
    rng = np.random.default_rng(K)
    n = 384
    sym = rng.integers(0, 1 << K, (4, n))
    lut = rng.standard_normal(1 << 16).astype(np.float16)
    got = o.decode(o.pack_symbols(sym, K), lut, n, K=K)
    for r in range(4):
        assert np.array_equal(_bits(got[r]), _bits(o.dequantize_symbols(lut, sym[r], K)))


def test_code_b_literal():
    # direct restatement of inference.cu:250-262 on a handful of windows
    rng = np.random.default_rng(5)
    lut = rng.standard_normal(512).astype(np.float16)
    sym = rng.integers(0, 16, (2, 64))
    got = o.decode(o.pack_symbols(sym, 4), lut, 128, code=o.CODE_B, S=8)
    for r in range(2):
        state = 0
        for s in range(64):
            state = ((state << 4) | int(sym[r, s])) & 0xFFFFFFFF
            h = (state * (state + 1)) & 0xFFFFFFFF
            e = (h >> 8) & 255
            lo = (int(lut[2 * e].view(np.uint16)) & 0x7FFF) | (h & 0x8000)
            assert int(got[r, 2 * s].view(np.uint16)) == lo
            assert got[r, 2 * s + 1].view(np.uint16) == lut[2 * e + 1].view(np.uint16)


def test_all_ones_codebook_gives_sum_of_x():
    # the known-answer idea of rptc_kernels/tests/test_decompress.py:11,38 (valid for code A)
    rng = np.random.default_rng(7)
    m, n = 32, 2048
    words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)
    lut = np.ones(1 << 16, dtype=np.float16)
    x = rng.standard_normal(n).astype(np.float16)
    y = o.matvec_exact(o.decode(words, lut, n), x[None])[0]
    assert np.allclose(y, x.astype(np.float64).sum())


def test_layout_round_trips_and_quirks():
    rng = np.random.default_rng(9)
    m, nu = 64, 64
    w = rng.integers(0, 2**32, (m, nu * 4), dtype=np.uint64).astype(np.uint32)
    for lay in (o.LAYOUT_ROWMAJOR, o.LAYOUT_CHUNKED, o.LAYOUT_UNITMAJOR, o.LAYOUT_TILED):
        assert np.array_equal(o.to_rowmajor(o.from_rowmajor(w, lay), lay), w)
    t = o.from_rowmajor(w, o.LAYOUT_TILED)
    assert t.shape == (m // 32, nu, 32, 4) and np.array_equal(t[1, 5, 7], w[32 + 7, 20:24])
    lut = rng.standard_normal(1 << 16).astype(np.float16)
    n = nu * 64
    strict = o.decode(w, lut, n)
    quirk = o.decode(w, lut, n, quirk=o.QUIRK_K1_LANE0_SEED)
    diff = np.nonzero((_bits(strict) != _bits(quirk)).any(axis=0))[0]
    # the defect of inference.cu:61-62 touches only columns c >= 2048 with c % 2048 < 7
    assert len(diff) > 0 and all(c >= 2048 and c % 2048 < 7 for c in diff)
    lutb = rng.standard_normal(512).astype(np.float16)
    sb = o.decode(w, lutb, n, code=o.CODE_B, S=8)
    qb = o.decode(w, lutb, n, code=o.CODE_B, S=8, quirk=o.QUIRK_K2_LANE0_CARRY)
    diffb = np.nonzero((_bits(sb) != _bits(qb)).any(axis=0))[0]
    assert len(diffb) > 0 and all(c % 2048 < 6 for c in diffb)


def test_k2_pair_source_is_a_permutation():
    for n in (2048, 4096, 8192):
        q = o.k2_pair_source(n)
        assert np.array_equal(np.sort(q), np.arange(n // 2))


def test_carry_in_equals_decoding_the_joined_stream():
    rng = np.random.default_rng(11)
    m, nu = 32, 8
    w = rng.integers(0, 2**32, (m, nu * 4), dtype=np.uint64).astype(np.uint32)
    lut = rng.standard_normal(512).astype(np.float16)
    full = o.decode(w, lut, nu * 64, code=o.CODE_B, S=8)
    right = o.decode(w[:, 16:], lut, (nu - 4) * 64, code=o.CODE_B, S=8, carry_in=w[:, 15])
    assert np.array_equal(_bits(full[:, 4 * 64:]), _bits(right))


@pytest.mark.parametrize("code,K,S,L", [(0, 2, 0, 16), (0, 3, 0, 16), (0, 4, 0, 16), (0, 2, 0, 14), (1, 2, 8, 16),
                                        (1, 2, 6, 16), (2, 2, 9, 16), (2, 4, 9, 16)])
def test_c_oracle_equals_numpy_oracle(code, K, S, L):
    rng = np.random.default_rng(100 + code * 10 + K)
    m, n = 64, 768
    w = rng.integers(0, 2**32, (m, n * K // 32), dtype=np.uint64).astype(np.uint32)
    if code == 0:
        lut = rng.standard_normal(1 << L).astype(np.float16)
    elif code == 1:
        lut = rng.standard_normal(2 << S).astype(np.float16)
    else:
        lut = rng.standard_normal((1 << S, 2)).astype(np.float16)
    ci = rng.integers(0, 65536, m).astype(np.uint32)
    ref = o.decode(w, lut, n, code=code, K=K, L=L, S=S, carry_in=ci)
    for lay in (o.LAYOUT_ROWMAJOR, o.LAYOUT_UNITMAJOR):
        got = c_oracle.decompress(o.from_rowmajor(w, lay), lut, m, n, code=code, K=K, L=L, S=S, layout=lay, carry_in=ci)
        assert np.array_equal(_bits(got), _bits(ref))
    x = rng.standard_normal((3, n)).astype(np.float16)
    y = c_oracle.gemv(w, lut, x, m, n, code=code, K=K, L=L, S=S, carry_in=ci)
    assert np.allclose(y, o.matvec_exact(ref, x), rtol=1e-4, atol=1e-3)


def test_rht_matches_scipy_hadamard():
    from scipy.linalg import hadamard
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 1024))
    s = o.signs_from_seed(5, 1024)
    H = np.kron(np.eye(4), hadamard(256)) / 16.0
    assert np.allclose(o.rht(x, s, 256), (x * s) @ H.T)
    assert np.allclose(o.rht(o.rht(x, s, 256), s, 256, transpose=True), x)
    assert o.hadamard_block(11008) == 256 and o.hadamard_block(4096) == 4096 and o.hadamard_block(28672) == 4096


@pytest.mark.parametrize("S", [8, 6])
def test_streams_built_for_the_reference_binary_pin_avoid_entries_below_eight(S):
    """The generator behind the exact pin of the HASH code against the compiled reference kernel (tests/test_gpu_legacy.py):
    under that kernel's own history rule no step may look up a table entry below 8."""
    from gpu_util import hash_entry, words_avoiding_low_entries
    n = 4096
    w = words_avoiding_low_entries(np.random.default_rng(S), 64, n, S)
    assert w.shape == (64, n // 16) and w.dtype == np.uint32
    win = o.windows(w, 4, n // 2, o.QUIRK_K2_LANE0_CARRY)
    assert (hash_entry(win, S) >= 8).all()
    assert abs(np.unpackbits(w.view(np.uint8)).mean() - 0.5) < 0.01          # still looks like a random stream
