"""CPU oracle for the RPTC decode + matvec hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy, what the reference computes for the path
"packed trellis bitstream -> shift-register state -> codebook / compute-code lookup ->
fp16 weights -> matvec".  It is the checker the CUDA kernels are compared against; nothing in
the product imports it.  Only the tests, the smoke check and the CPU-baseline leg of the
benchmark may call it.

Pin status: the reference ships no golden vectors or asserting tests for this path
(rptc_kernels/tests/*.py only print).  The oracle is therefore pinned two ways:
  * known-answer patterns taken from the reference's own scripts (all-ones codebook gives
    out == sum(x), rptc_kernels/tests/test_decompress.py:11,38), plus hand-derived vectors in
    tests/golden/;
  * on a GPU box, against the UNMODIFIED reference extension compiled by oracle/build_ref.sh
    (`refkernel` mode below reproduces the reference kernels including their lane-0 quirks,
    so every element can be compared).

Codes (reference file:line each follows):
  code A  "LUT"      rptc.py:74-85          s=((s<<K)|q)&(2^L-1), w=alphabet[s]; bit order of the
                                            packed words from inference.cu:66-94 (MSB first).
  code B  "hash"     inference.cu:237-263   4 bits/step, 2 weights/step, t(t+1) hash, entry bits
                                            8..8+S, sign of the low half from hash bit 15.
  code C  "lite"     rptc_lite.py:12-16,63-73  h=x(2x+1); h^=h>>(L-S); idx=h&(2^S-1); V=2.

Layouts of the packed words (all int32/uint32, 128-bit "units" of 4 words):
  ROWMAJOR  [m, n_units*4]          inference.cu:53-66   (decompress_kernel)
  CHUNKED   [n_units/32, m, 32*4]   inference.cu:229     (decompress_matvec_kernel; lane-major)
  UNITMAJOR [n_units, m, 4]         inference_t.cu:116   (decompress_matvec_t_kernel)
  TILED     [m/32, n_units, 32, 4]  the native layout of the B200 kernels (no reference counterpart)
"""
from __future__ import annotations

import numpy as np

CODE_A = 0   # LUT code, K bits per weight, one weight per step
CODE_B = 1   # reference fused-kernel hash code, 4 bits per step, two weights per step
CODE_C = 2   # rptc_lite compute-code, R bits per step, two weights per step

LAYOUT_ROWMAJOR = 0
LAYOUT_CHUNKED = 1
LAYOUT_UNITMAJOR = 2
LAYOUT_TILED = 3

QUIRK_NONE = 0
QUIRK_K1_LANE0_SEED = 1    # inference.cu:61-62: lane 0 seeds from the HIGH half of the previous word
QUIRK_K2_LANE0_CARRY = 2   # inference.cu:232: lane 0's carry is its own .w, not the previous lane-31 .w

# Order in which the fused reference kernel's eight 32-bit window registers are met along the
# stream (inference.cu:237-243): reg_c[7] holds carry:x.hi, reg_c[0]=x, reg_c[4]=x.lo:y.hi, ...
K2_WINDOW_ORDER = (7, 0, 4, 1, 5, 2, 6, 3)


# ----------------------------------------------------------------------------------------------
# layouts
# ----------------------------------------------------------------------------------------------
def to_rowmajor(words: np.ndarray, layout: int) -> np.ndarray:
    """Any supported layout -> ROWMAJOR [m, n_units*4] uint32."""
    w = np.ascontiguousarray(words).view(np.uint32)
    if layout == LAYOUT_ROWMAJOR:
        assert w.ndim == 2 and w.shape[1] % 4 == 0
        return w
    if layout == LAYOUT_CHUNKED:
        iters, m, k = w.shape
        assert k == 128
        return np.ascontiguousarray(w.transpose(1, 0, 2).reshape(m, iters * 128))
    if layout == LAYOUT_UNITMAJOR:
        nu, m, k = w.shape
        assert k == 4
        return np.ascontiguousarray(w.transpose(1, 0, 2).reshape(m, nu * 4))
    if layout == LAYOUT_TILED:
        nrb, nu, lanes, k = w.shape
        assert lanes == 32 and k == 4
        return np.ascontiguousarray(w.transpose(0, 2, 1, 3).reshape(nrb * 32, nu * 4))
    raise ValueError(f"unknown layout {layout}")


def from_rowmajor(words: np.ndarray, layout: int) -> np.ndarray:
    """ROWMAJOR [m, n_units*4] uint32 -> the requested layout."""
    w = np.ascontiguousarray(words).view(np.uint32)
    m, nw = w.shape
    assert nw % 4 == 0
    nu = nw // 4
    if layout == LAYOUT_ROWMAJOR:
        return w
    if layout == LAYOUT_CHUNKED:
        assert nu % 32 == 0, "CHUNKED needs a multiple of 32 units (2048 weights at 2 bits) per row"
        return np.ascontiguousarray(w.reshape(m, nu // 32, 128).transpose(1, 0, 2))
    if layout == LAYOUT_UNITMAJOR:
        return np.ascontiguousarray(w.reshape(m, nu, 4).transpose(1, 0, 2))
    if layout == LAYOUT_TILED:
        assert m % 32 == 0
        return np.ascontiguousarray(w.reshape(m // 32, 32, nu, 4).transpose(0, 2, 1, 3))
    raise ValueError(f"unknown layout {layout}")


# ----------------------------------------------------------------------------------------------
# bitstream windows
# ----------------------------------------------------------------------------------------------
def _halfwords(words_rm: np.ndarray) -> np.ndarray:
    """[m, nw] uint32 -> [m, 2*nw] uint32 of 16-bit halfwords in stream (MSB-first) order."""
    w = words_rm.astype(np.uint32)
    h = np.empty((w.shape[0], w.shape[1] * 2), dtype=np.uint32)
    h[:, 0::2] = w >> 16
    h[:, 1::2] = w & 0xFFFF
    return h


def windows(words_rm: np.ndarray, bits_per_step: int, n_steps: int, quirk: int = QUIRK_NONE,
            carry_in: np.ndarray | None = None) -> np.ndarray:
    """The 16-bit window of the row's bitstream that ends with step s, for every s.

    Step s consumes bits [s*b, (s+1)*b) of the row (b = bits_per_step); the shift-register state
    after it is the last 16 bits seen, zero-filled before the row start (rptc.py:77-83,
    init_state = 0; inference.cu:57-59).  `carry_in` ([m] uint, low 16 bits used) replaces the zero
    fill: it is the halo a column-sharded tensor carries over from the shard on its left.
    Returns [m, n_steps] uint32 with values < 65536.
    """
    h = _halfwords(words_rm)
    m, nh = h.shape
    assert n_steps * bits_per_step <= nh * 16, "stream shorter than the requested steps"
    e = (np.arange(n_steps, dtype=np.int64) + 1) * bits_per_step    # end bit (exclusive), 1-based count
    g = (e - 1) // 16                                               # halfword holding the last bit
    shift = (16 * (g + 1) - e).astype(np.uint32)                    # 0..15
    cur = h[:, g]
    prev = np.zeros_like(cur)
    nz = g > 0
    prev[:, nz] = h[:, g[nz] - 1]
    if carry_in is not None:
        ci = (np.asarray(carry_in).astype(np.uint32) & 0xFFFF)[:, None]
        prev[:, ~nz] = ci
    if quirk != QUIRK_NONE:
        # a 128-bit unit is 8 halfwords; units whose index is a multiple of 32 are "lane 0"
        lane0 = (g % 256 == 0)
        if quirk == QUIRK_K1_LANE0_SEED:
            sel = lane0 & (g > 0)
            prev[:, sel] = h[:, g[sel] - 2]          # high half of the previous unit's last word
        elif quirk == QUIRK_K2_LANE0_CARRY:
            sel = lane0
            prev[:, sel] = h[:, g[sel] + 7]          # low half of the unit's own last word
        else:
            raise ValueError(f"unknown quirk {quirk}")
    win = ((prev << np.uint32(16)) | cur) >> shift[None, :]
    return win & np.uint32(0xFFFF)


# ----------------------------------------------------------------------------------------------
# state -> weights
# ----------------------------------------------------------------------------------------------
def hash_b(t: np.ndarray) -> np.ndarray:
    """inference.cu:250-251: hash = t*(t+1) in uint32; only its low 16 bits are ever used."""
    t = t.astype(np.uint64)
    return ((t * (t + 1)) & 0xFFFF).astype(np.uint32)


def index_c(t: np.ndarray, L: int, S: int) -> np.ndarray:
    """rptc_lite.py:12-16 on the low L bits of the state (the result depends on nothing else)."""
    x = t.astype(np.uint64) & ((1 << L) - 1)
    h = (x * (2 * x + 1)) & ((1 << L) - 1)
    h ^= h >> (L - S)
    return (h & ((1 << S) - 1)).astype(np.uint32)


def decode(words: np.ndarray, lut: np.ndarray, n: int, code: int = CODE_A, K: int = 2, L: int = 16,
           S: int = 8, layout: int = LAYOUT_ROWMAJOR, quirk: int = QUIRK_NONE,
           carry_in: np.ndarray | None = None) -> np.ndarray:
    """Packed codes -> dense fp16 [m, n], bit-exact.

    code A: `lut` is fp16 [2^L]; K bits per weight.
    code B: `lut` is fp16 [2^(S+1)] read as 2^S (lo, hi) pairs (inference.cu:303-306); 2 bits/weight.
    code C: `lut` is fp16 [2^S, 2]; K bits per weight, R = 2K bits per step.
    Column order is stream order: step s yields column s (code A) or columns 2s, 2s+1 (B, C).
    """
    rm = to_rowmajor(words, layout)
    lut16 = np.ascontiguousarray(lut, dtype=np.float16)
    if code == CODE_A:
        assert lut16.size == 1 << L
        win = windows(rm, K, n, quirk, carry_in) & np.uint32((1 << L) - 1)
        return lut16.reshape(-1)[win]
    assert n % 2 == 0
    if code == CODE_B:
        assert K == 2 and lut16.size == 2 << S
        win = windows(rm, 4, n // 2, quirk, carry_in)
        h = hash_b(win)
        pairs = lut16.reshape(-1, 2)[(h >> 8) & ((1 << S) - 1)]          # [m, n/2, 2]
        bits = pairs.view(np.uint16).copy()
        bits[..., 0] = (bits[..., 0] & 0x7FFF) | (h & 0x8000).astype(np.uint16)   # inference.cu:258-262
        return bits.view(np.float16).reshape(rm.shape[0], n)
    if code == CODE_C:
        assert lut16.shape == (1 << S, 2)
        win = windows(rm, 2 * K, n // 2, quirk, carry_in)
        return lut16[index_c(win, L, S)].reshape(rm.shape[0], n)
    raise ValueError(f"unknown code {code}")


def dequantize_symbols(alphabet: np.ndarray, quantized: np.ndarray, K: int = 2) -> np.ndarray:
    """Literal restatement of rptc.py:74-85 (one row, sequential scan) for cross-checking `decode`."""
    M = alphabet.shape[0]
    state = 0
    out = np.empty(len(quantized), dtype=alphabet.dtype)
    for i, q in enumerate(quantized):
        state = (M - 1) & ((state << K) | int(q))
        out[i] = alphabet[state]
    return out


def dequantize_lite_symbols(alphabet: np.ndarray, L: int, S: int, R: int, quantized: np.ndarray) -> np.ndarray:
    """Literal restatement of rptc_lite.py:63-73 with int32 wrap-around, one row."""
    state = 0
    out = np.empty((len(quantized), alphabet.shape[1]), dtype=alphabet.dtype)
    for i, q in enumerate(quantized):
        state = _wrap32((state << R) | int(q))
        x = _wrap32(state * (2 * state + 1))
        x ^= x >> (L - S)                      # Python's >> on a negative int is arithmetic, like int32
        out[i] = alphabet[x & ((1 << S) - 1)]
    return out


def _wrap32(v: int) -> int:
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v & 0x80000000 else v


def pack_symbols(symbols: np.ndarray, bits: int) -> np.ndarray:
    """[m, T] symbols (each < 2^bits) -> ROWMAJOR uint32 words, MSB first (inference.cu:70-71).

    The row is zero-padded up to a whole number of 128-bit units.
    """
    sym = np.asarray(symbols).astype(np.uint64)
    m, T = sym.shape
    total = T * bits
    nw = -(-total // 128) * 4
    stream = np.zeros((m, nw * 32), dtype=np.uint8)
    for b in range(bits):
        stream[:, b:total:bits] = ((sym >> np.uint64(bits - 1 - b)) & np.uint64(1)).astype(np.uint8)
    weights = (np.uint64(1) << np.arange(31, -1, -1, dtype=np.uint64))
    return (stream.reshape(m, nw, 32).astype(np.uint64) * weights).sum(axis=2).astype(np.uint32)


# ----------------------------------------------------------------------------------------------
# matvec
# ----------------------------------------------------------------------------------------------
def k2_pair_source(n: int) -> np.ndarray:
    """x-pair read by each stream step in the fused reference kernel (inference.cu:216-221,249).

    Returns q[s] for s in [0, n/2): step s of the row's stream multiplies x[2q], x[2q+1].
    """
    assert n % 2048 == 0
    iters = n // 2048
    q = np.empty(n // 2, dtype=np.int64)
    lane = np.arange(32)
    for it in range(iters):
        for o, k in enumerate(K2_WINDOW_ORDER):
            for j in range(4):
                p = ((it * 8 + k) * 4 + j) * 32 + lane
                s = (it * 32 + lane) * 32 + o * 4 + j
                q[s] = 4 * (p % (n // 8)) + p // (n // 8)
    return q


def permute_x_k2(x: np.ndarray) -> np.ndarray:
    """x as the fused reference kernel pairs it with the stream: x'[2s:2s+2] = x[2q[s]:2q[s]+2]."""
    x = np.asarray(x)
    n = x.shape[-1]
    q = k2_pair_source(n)
    return x.reshape(*x.shape[:-1], n // 2, 2)[..., q, :].reshape(x.shape)


def matvec_exact(w16: np.ndarray, x16: np.ndarray) -> np.ndarray:
    """fp64 product of fp16 weights [m, n] and fp16 activations [b, n] -> [b, m] float64."""
    return np.asarray(x16, dtype=np.float64) @ np.asarray(w16, dtype=np.float64).T


def _f16(a):
    return np.asarray(a, dtype=np.float64).astype(np.float16)


def matvec_k2_fp16(words_chunked: np.ndarray, lut: np.ndarray, x: np.ndarray, S: int,
                   quirk: int = QUIRK_K2_LANE0_CARRY) -> np.ndarray:
    """Emulates decompress_matvec_kernel's fp16 arithmetic (inference.cu:228-276) step for step:
    per-lane half2 HFMA2 accumulation in loop order (iter, k, j), shuffle-down tree in fp16,
    then x+y.  Each fp16 operation is computed in float64 and rounded once, which equals the fused
    fp16 result except on measure-zero double-rounding ties.
    """
    iters, m, _ = words_chunked.shape
    n = iters * 2048
    w = decode(words_chunked, lut, n, code=CODE_B, S=S, layout=LAYOUT_CHUNKED, quirk=quirk)   # [m, n] stream order
    xs = permute_x_k2(np.asarray(x, dtype=np.float16))                                       # stream order
    wq = w.reshape(m, iters, 32, 8, 4, 2).astype(np.float64)      # [m, iter, lane, order-pos, j, half]
    xq = xs.reshape(iters, 32, 8, 4, 2).astype(np.float64)
    acc = np.zeros((m, 32, 2), dtype=np.float16)
    pos_of_k = {k: o for o, k in enumerate(K2_WINDOW_ORDER)}
    for it in range(iters):
        for k in range(8):
            o = pos_of_k[k]
            for j in range(4):
                acc = _f16(wq[:, it, :, o, j, :] * xq[None, it, :, o, j, :] + acc.astype(np.float64))
    off = 16
    while off:
        nxt = acc.copy()
        nxt[:, : 32 - off] = _f16(acc[:, : 32 - off].astype(np.float64) + acc[:, off:].astype(np.float64))
        acc = nxt
        off //= 2
    return _f16(acc[:, 0, 0].astype(np.float64) + acc[:, 0, 1].astype(np.float64))


def matvec_k3_as_written(words_unitmajor: np.ndarray, lut: np.ndarray, x: np.ndarray, out_init: np.ndarray,
                         L: int = 16) -> np.ndarray:
    """What decompress_matvec_t_kernel computes AS WRITTEN (inference_t.cu:112-171), fp16 step for
    step: within each 32-bit word the shift registers are not advanced between the eight j
    iterations, so the word's first two weights are used eight times, against act[col*32+k*8+j].
    """
    nu, m, _ = words_unitmajor.shape
    mask = (1 << L) - 1
    cb = np.asarray(lut, dtype=np.float16).reshape(-1)
    xp = np.asarray(x, dtype=np.float16).reshape(-1, 2).astype(np.float64)
    words = words_unitmajor.view(np.uint32).astype(np.uint64)
    carries = np.zeros(m, dtype=np.uint64)
    acc = np.zeros((m, 2), dtype=np.float16)
    for col in range(nu):
        for k in range(4):
            wd = words[col, :, k]
            s2 = (((carries << np.uint64(2)) | (wd >> np.uint64(30))) & np.uint64(0xFFFFFFFF)) & np.uint64(mask)
            s4 = (((carries << np.uint64(4)) | (wd >> np.uint64(28))) & np.uint64(0xFFFFFFFF)) & np.uint64(mask)
            carries = s4
            wpair = np.stack([cb[s2.astype(np.int64)], cb[s4.astype(np.int64)]], axis=1).astype(np.float64)
            for j in range(8):
                acc = _f16(wpair * xp[None, col * 32 + k * 8 + j, :] + acc.astype(np.float64))
    delta = _f16(acc[:, 0].astype(np.float64) + acc[:, 1].astype(np.float64))
    return _f16(np.asarray(out_init, dtype=np.float16).astype(np.float64) + delta.astype(np.float64))


# ----------------------------------------------------------------------------------------------
# randomized Hadamard transform (extension of this build; no counterpart in the reference)
# ----------------------------------------------------------------------------------------------
def hadamard_block(n: int) -> int:
    """Largest power of two dividing n, capped at 4096: the block size of the block-diagonal transform."""
    b = n & (-n)
    return min(b, 4096)


def rht(x: np.ndarray, signs: np.ndarray, block: int, transpose: bool = False) -> np.ndarray:
    """Block-diagonal randomized Hadamard transform along the last axis, in float64.

    forward   : y = H_b (s * x) / sqrt(b)   per block of `block` elements
    transpose : y = s * (H_b x) / sqrt(b)   (H is symmetric, so this is the inverse of forward)
    H_b is the Sylvester (natural-order) Hadamard matrix; s = +-1.
    """
    x = np.asarray(x, dtype=np.float64)
    n = x.shape[-1]
    assert n % block == 0 and block & (block - 1) == 0
    s = np.asarray(signs, dtype=np.float64)
    y = (x if transpose else x * s).reshape(-1, block)
    h = 1
    while h < block:
        y = y.reshape(-1, block // (2 * h), 2, h)
        y = np.stack([y[:, :, 0, :] + y[:, :, 1, :], y[:, :, 0, :] - y[:, :, 1, :]], axis=2).reshape(-1, block)
        h *= 2
    y = y.reshape(x.shape) / np.sqrt(block)
    return y * s if transpose else y


def signs_from_seed(seed: int, n: int) -> np.ndarray:
    """+-1 vector from a 64-bit seed: bit i of a SplitMix64 stream (one word per 64 elements)."""
    out = np.empty(n, dtype=np.float32)
    mask = (1 << 64) - 1
    state = seed & mask
    for w in range(-(-n // 64)):
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        for b in range(min(64, n - 64 * w)):
            out[64 * w + b] = -1.0 if (z >> b) & 1 else 1.0
    return out
