"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import rptc_oracle as o


def rand_words(rng, m, n, K):
    return rng.integers(0, 2**32, (m, n * K // 32), dtype=np.uint64).astype(np.uint32)


def rand_lut(rng, code, L=16, S=8):
    if code == o.CODE_A:
        return rng.standard_normal(1 << L).astype(np.float16)
    return rng.standard_normal(2 << S).astype(np.float16)


def to_dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).cuda()


def bits(a):
    if isinstance(a, torch.Tensor):
        a = a.cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def lut_for_oracle(lut, code, S):
    return lut.reshape(1 << S, 2) if code == o.CODE_C else lut


# ---- tolerances derived from the kernels' arithmetic --------------------------------------------------------
# |w|, |x| below are the Euclidean norms of a weight row and an activation row; y is the exact product.
#  * batch 1 (HFMA2 kernels): four fp16 accumulators per 64-weight unit take eight fp16 products each, three fp16
#    adds join them, everything after that is fp32.  Each fp16 rounding is 2^-11 of a partial sum of at most 64
#    terms, and the roundings of the n/64 units add in quadrature: about 4e-5 |w||x| at the worst row of a
#    4096 x 4096 layer (0.147 absolute measured).  Bound: 1.5e-4 |w||x|.
#  * batch >= 2 (mma.sync kernel) and the tcgen05 GEMM: fp16 products summed in fp32.  Bound: 2e-5 |w||x|.
#  * the fp16 rounding of the result itself: 2^-11 |y|.
# One mis-decoded weight moves an output by |dw * x_c|, about 1 for N(0,1) weights and activations: at n = 4096 the
# batch-1 bound is 0.6 absolute and the others 0.08, against 8.2 for the bound these tests used before.
GEMV_HFMA2_TOL = 1.5e-4
GEMV_FP32_TOL = 2e-5


def check_product(y, exact, wnorm, xnorm, rel, what=""):
    """y, exact: [b, m] float64 arrays; wnorm [m], xnorm [b].  Returns max err/tol (also printed)."""
    err = np.abs(np.asarray(y, dtype=np.float64) - exact)
    tol = rel * wnorm[None, :] * xnorm[:, None] + 2.0**-11 * np.abs(exact) + 1e-4
    worst = float(np.max(err / tol))
    print(f"{what} max err {err.max():.4g}, max err/tol {worst:.3f}")
    assert worst <= 1.0, f"{what} max err/tol {worst:.3f}"
    return worst


def probe_columns(run, n, batch, m, cols=None):
    """Exact-column probing: run(x) -> y for x fp16 [batch, n] whose rows are unit vectors.  Every product is then a
    weight times one or zero and every partial sum a weight plus zeros, exact in fp16 and fp32, so the output row of
    column c must equal column c of the decoded matrix bit for bit.  Returns Y [len(cols), m] fp16 (all columns when
    `cols` is None)."""
    cols = torch.arange(n, device="cuda") if cols is None else torch.as_tensor(cols, device="cuda", dtype=torch.long)
    Y = torch.empty((len(cols), m), dtype=torch.float16, device="cuda")
    x = torch.zeros((batch, n), dtype=torch.float16, device="cuda")
    ar = torch.arange(batch, device="cuda")
    for i0 in range(0, len(cols), batch):
        c = cols[i0:i0 + batch]
        k = len(c)
        x.zero_()
        x[ar[:k], c] = 1.0
        Y[i0:i0 + k] = run(x)[:k]
    return Y


def assert_same_bits(a, b, what=""):
    """Two fp16 CUDA tensors, compared as raw 16-bit patterns."""
    a, b = a.contiguous().view(torch.int16), b.contiguous().view(torch.int16)
    if not torch.equal(a, b):
        bad = (a != b).nonzero()
        raise AssertionError(f"{what}: {len(bad)} of {a.numel()} elements differ, first at {bad[0].tolist()}")


def hash_entry(t, S):
    """Table entry the fused reference kernel looks up for window t (inference.cu:250-257)."""
    t = t.astype(np.uint64)
    return (((t * (t + 1)) >> np.uint64(8)) & np.uint64((1 << S) - 1)).astype(np.int64)


def words_avoiding_low_entries(rng, m, n, S, lowest=8):
    """Row-major stream words [m, n/16] in which NO step of the fused reference kernel looks up a table entry below
    `lowest`, under that kernel's own history rule (every 32nd unit takes its own last word as carry, inference.cu:232;
    this includes the first unit of a row, so even a row's first windows are not the near-zero ones).

    Any bitstream is a valid trellis path, so the row is walked greedily: each 4-bit symbol is drawn (random order of
    the 16 candidates) among those whose 16-bit window is `alive`: its entry is >= lowest and it has an alive successor
    (the greatest such set, by pruning).  In a unit with the carry deviation the first three windows hold the unit's
    LAST 16 bits; such a unit is redrawn until they comply."""
    states = np.arange(1 << 16, dtype=np.uint32)
    alive = hash_entry(states, S) >= lowest
    succ = ((states[:, None] << 4) | np.arange(16, dtype=np.uint32)[None, :]) & 0xFFFF
    while True:
        pruned = alive & alive[succ].any(axis=1)
        if (pruned == alive).all():
            break
        alive = pruned
    assert alive.mean() > 0.5
    nu = n // 64
    nib = np.zeros((m, nu, 32), dtype=np.uint32)
    hist = np.zeros(m, dtype=np.uint32)
    for u in range(nu):
        lane0 = u % 32 == 0
        todo = np.ones(m, dtype=bool)
        new_hist = hist.copy()
        for _ in range(500):
            idx = np.nonzero(todo)[0]
            if len(idx) == 0:
                break
            k = len(idx)
            h = hist[idx].copy()
            nb = np.zeros((k, 32), dtype=np.uint32)
            good = np.ones(k, dtype=bool)
            start = 0
            if lane0:                                  # checked at the end, against the unit's own last 16 bits
                for s in range(3):
                    nb[:, s] = rng.integers(0, 16, k)
                    h = ((h << 4) | nb[:, s]) & 0xFFFF
                start = 3
            for s in range(start, 32):
                cand = (rng.integers(0, 16, k)[:, None] + np.arange(16)[None, :]).astype(np.uint32) % 16
                t = ((h[:, None] << 4) | cand) & 0xFFFF
                ok = alive[t]
                good &= ok.any(axis=1)                 # a dead end can only follow the three free symbols of a lane-0 unit
                pick = ok.argmax(axis=1)
                nb[:, s] = cand[np.arange(k), pick]
                h = t[np.arange(k), pick]
            if lane0:
                hq = h.copy()
                for s in range(3):
                    hq = ((hq << 4) | nb[:, s]) & 0xFFFF
                    good &= hash_entry(hq, S) >= lowest
            nib[idx[good], u] = nb[good]
            new_hist[idx[good]] = h[good]
            todo[idx[good]] = False
        assert not todo.any()
        hist = new_hist
    shifts = np.arange(28, -4, -4, dtype=np.uint32)
    words = (nib.reshape(m, nu, 4, 8) << shifts[None, None, None, :]).sum(axis=3, dtype=np.uint64).astype(np.uint32)
    return words.reshape(m, nu * 4)
