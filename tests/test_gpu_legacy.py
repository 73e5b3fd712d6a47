"""GPU parity of the drop-in `rptc_kernels` module: against the CPU oracle, and (when oracle/_ref holds
the compiled, unmodified reference extension) against the reference's own kernels on the same
inputs.  The reference runs in a child process (see tests/ref_runner.py)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import rptc_oracle as o
from gpu_util import GEMV_HFMA2_TOL, bits, check_product, hash_entry, to_dev, words_avoiding_low_entries

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run_reference(which, m, n, seed, tmp_path, words=None):
    path = str(tmp_path / f"{which}.npz")
    cmd = [sys.executable, os.path.join(HERE, "ref_runner.py"), which, path, str(m), str(n), str(seed)]
    if words is not None:
        np.save(str(tmp_path / "words.npy"), words)
        cmd.append(str(tmp_path / "words.npy"))
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if r.returncode == 3:
        pytest.skip("oracle/_ref reference extension not built")
    # the extension exists: anything but success is a lost pin, not a reason to skip
    assert r.returncode == 0, f"the reference extension failed (exit {r.returncode}): {r.stdout[-300:]} {r.stderr[-600:]}"
    return np.load(path)


def test_reference_decompress_pins_oracle_and_drop_in(tmp_path):
    import rptc_kernels
    m, n = 64, 6144
    d = _run_reference("decompress", m, n, 1, tmp_path)
    ref_out = d["out"]
    # (1) the oracle in refkernel mode reproduces the reference kernel on EVERY element
    assert np.array_equal(bits(o.decode(d["words"], d["lut"], n, quirk=o.QUIRK_K1_LANE0_SEED)), bits(ref_out))
    # (2) so does the drop-in with the quirk switched on
    out = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    rptc_kernels.set_reference_quirks(True)
    try:
        ms = rptc_kernels.decompress(to_dev(d["words"]), to_dev(d["lut"]), out)
    finally:
        rptc_kernels.set_reference_quirks(False)
    assert isinstance(ms, float) and ms > 0
    assert np.array_equal(bits(out), bits(ref_out))
    # (3) and the default (self-consistent) decode differs only where inference.cu:61-62 reads the wrong half
    rptc_kernels.decompress(to_dev(d["words"]), to_dev(d["lut"]), out)
    diff = np.nonzero((bits(out) != bits(ref_out)).any(axis=0))[0]
    assert all(c >= 2048 and c % 2048 < 7 for c in diff)
    assert np.array_equal(bits(out), bits(o.decode(d["words"], d["lut"], n)))


@pytest.mark.parametrize("S,n", [(8, 2048), (8, 4096), (6, 2048), (6, 8192)])
def test_reference_fused_matvec_pins_the_hash_code(tmp_path, S, n):
    """The HASH code pinned to the reference binary, exactly.

    The compiled decompress_matvec_16_{6,8}_1 splices the table entry into bits 7.. of a shared-memory pointer and
    relies on its table starting at a 32 KiB-aligned shared address (inference.cu:206,252-257).  Where the first KiB of
    the shared window is reserved the table starts at 0x400, bit 10 of the base is overwritten by the splice, and entry e
    answers with entry e - 8; entries 0..7 read reserved memory.  On streams in which no step looks up an entry below 8
    the kernel is therefore the oracle's step-for-step fp16 emulation run with the table moved up by eight entries
    -- and if the table does sit on its boundary, with the table as it is.  Either way window order (7,0,4,1,5,2,6,3),
    hash, entry bits, sign bit, lane-0 carry and the activation permutation (inference.cu:216-221,232,237-263) must
    all be right for the outputs to agree to the last fp16 bit."""
    m = 128
    rng = np.random.default_rng(100 + S + n)
    words = words_avoiding_low_entries(rng, m, n, S)
    win = o.windows(words, 4, n // 2, o.QUIRK_K2_LANE0_CARRY)
    assert (hash_entry(win, S) >= 8).all()
    d = _run_reference(f"matvec_16_{S}_1", m, n, 2 + S, tmp_path, words=words)
    assert np.array_equal(d["words"], words)
    ref_out = d["out"].astype(np.float64)
    chunked = o.from_rowmajor(words, o.LAYOUT_CHUNKED)
    pairs = d["lut"].reshape(-1, 2)
    displaced = np.zeros_like(pairs)
    displaced[8:] = pairs[:-8]              # entry e answers with entry e-8; entries 0..7 are never looked up here
    ulp = np.maximum(np.abs(ref_out), 1.0) * 2.0**-10
    verdicts = {}
    for name, table in (("table moved up by 8 entries", displaced.reshape(-1)), ("table in place", d["lut"])):
        emu = o.matvec_k2_fp16(chunked, table, d["x"], S).astype(np.float64)
        verdicts[name] = (float(np.max(np.abs(emu - ref_out) / ulp)), float(np.mean(emu == ref_out)))
    best = min(verdicts.values(), key=lambda v: v[0])
    print(f"S={S} n={n}: " + "; ".join(f"{k}: max {v[0]:.2f} ulp, {100 * v[1]:.1f} % identical" for k, v in verdicts.items()))
    assert best[0] <= 2.0 and best[1] > 0.9, verdicts


@pytest.mark.parametrize("S", [8, 6])
def test_reference_fused_matvec_against_oracle_emulation(tmp_path, S):
    """The fused reference kernel splices table-entry bits into the low 32 bits of a shared-memory
    pointer and relies on its table starting at a 32 KiB-aligned shared address (inference.cu:206,
    252-257).  Where the first KiB of the shared window is reserved by the system the table starts at
    0x400 instead, every lookup lands 8 entries low, and lookups of entries 0..7 read reserved
    memory.  The test accepts either outcome and says which one it saw: an exact match with the
    oracle's step-for-step fp16 emulation (then the pin holds), or the displaced-table signature."""
    m, n = 128, 4096
    d = _run_reference(f"matvec_16_{S}_1", m, n, 2 + S, tmp_path)
    ref_out = d["out"].astype(np.float64)
    chunked = o.from_rowmajor(d["words"], o.LAYOUT_CHUNKED)
    emu = o.matvec_k2_fp16(chunked, d["lut"], d["x"], S).astype(np.float64)
    ulp = np.maximum(np.abs(ref_out), 1.0) * 2.0**-10
    if (np.abs(emu - ref_out) <= 2 * ulp).all():
        assert np.mean(emu == ref_out) > 0.9
        return
    pairs = d["lut"].reshape(-1, 2)
    displaced = np.zeros_like(pairs)
    displaced[8:] = pairs[:-8]              # entry e now answers with entry e-8; 0..7 are unknown (zero here)
    emu_d = o.matvec_k2_fp16(chunked, displaced.reshape(-1), d["x"], S).astype(np.float64)
    corr_plain = np.corrcoef(emu, ref_out)[0, 1]
    corr_disp = np.corrcoef(emu_d, ref_out)[0, 1]
    assert corr_disp > 0.9 and corr_disp > corr_plain + 0.3, (corr_plain, corr_disp)
    pytest.skip(f"reference fused kernel reads its table 1 KiB low on this GPU (corr with displaced-table "
                f"emulation {corr_disp:.3f}, with the intended table {corr_plain:.3f}); not usable as a pin")


@pytest.mark.parametrize("S", [8, 6])
def test_drop_in_fused_matvec_quirk_mode_against_oracle(S):
    import rptc_kernels
    rng = np.random.default_rng(2 + S)
    m, n = 128, 4096
    words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)
    x = rng.standard_normal(n).astype(np.float16)
    lut = rng.standard_normal(2 << S).astype(np.float16)
    chunked = o.from_rowmajor(words, o.LAYOUT_CHUNKED)
    out = torch.zeros((m,), dtype=torch.float16, device="cuda")
    fn = getattr(rptc_kernels, f"decompress_matvec_16_{S}_1")
    rptc_kernels.set_reference_quirks(True)
    try:
        fn(to_dev(chunked), to_dev(lut), to_dev(x), out)
    finally:
        rptc_kernels.set_reference_quirks(False)
    w16 = o.decode(chunked, lut, n, code=o.CODE_B, S=S, layout=o.LAYOUT_CHUNKED, quirk=o.QUIRK_K2_LANE0_CARRY)
    exact = o.matvec_exact(w16, o.permute_x_k2(x)[None])[0]
    scale = np.linalg.norm(w16.astype(np.float64), axis=1) * np.linalg.norm(x.astype(np.float64))
    ours = out.float().cpu().numpy().astype(np.float64)
    check_product(ours[None], exact[None], np.linalg.norm(w16.astype(np.float64), axis=1), np.array([np.linalg.norm(x.astype(np.float64))]),
                  GEMV_HFMA2_TOL, f"quirk-mode drop-in S={S}")
    # the fp16 emulation of the reference's accumulation sits inside a much wider band around the same product
    emu = o.matvec_k2_fp16(chunked, lut, x, S).astype(np.float64)
    assert (np.abs(emu - exact) <= 3e-2 * scale).all()
    assert np.abs(ours - exact).mean() <= np.abs(emu - exact).mean()


def test_reference_transposed_matvec_as_written_pins_oracle(tmp_path):
    m, n = 256, 1024
    d = _run_reference("matvec_t_16", m, n, 5, tmp_path)
    um = o.from_rowmajor(d["words"], o.LAYOUT_UNITMAJOR)
    emu = o.matvec_k3_as_written(um, d["lut"], d["x"], d["init"]).astype(np.float64)
    ref_out = d["out"].astype(np.float64)
    ulp = np.maximum(np.abs(ref_out), 1.0) * 2.0**-10
    assert (np.abs(emu - ref_out) <= 2 * ulp).all()


def test_legacy_fused_matvec_strict_against_oracle():
    import rptc_kernels
    rng = np.random.default_rng(81)
    m, n = 256, 8192
    words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)
    chunked = o.from_rowmajor(words, o.LAYOUT_CHUNKED)
    x = rng.standard_normal(n).astype(np.float16)
    for S, names in ((8, ("decompress_matvec_16_8_1", "decompress_matvec_20_8_1")),
                     (6, ("decompress_matvec_16_6_1", "decompress_matvec_20_6_1"))):
        lut = rng.standard_normal(2 << S).astype(np.float16)
        w16 = o.decode(words, lut, n, code=o.CODE_B, S=S)
        exact = o.matvec_exact(w16, o.permute_x_k2(x)[None])[0]
        scale = np.linalg.norm(w16.astype(np.float64), axis=1) * np.linalg.norm(x.astype(np.float64))
        for name in names:
            out = torch.full((m,), 3.0, dtype=torch.float16, device="cuda")     # overwritten, not accumulated
            ms = getattr(rptc_kernels, name)(to_dev(chunked), to_dev(lut), to_dev(x), out)
            assert ms > 0
            check_product(out.float().cpu().numpy()[None], exact[None], np.linalg.norm(w16.astype(np.float64), axis=1),
                          np.array([np.linalg.norm(x.astype(np.float64))]), GEMV_HFMA2_TOL, name)


@pytest.mark.parametrize("L", [16, 14])
def test_legacy_transposed_matvec_intended_semantics(L):
    import rptc_kernels
    rng = np.random.default_rng(91 + L)
    m, n = 256, 4096
    words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)
    um = o.from_rowmajor(words, o.LAYOUT_UNITMAJOR)
    lut = rng.standard_normal(1 << L).astype(np.float16)
    x = rng.standard_normal(n).astype(np.float16)
    init = rng.standard_normal(m).astype(np.float16)
    out = to_dev(init.copy())
    fn = getattr(rptc_kernels, f"decompress_matvec_t_{L}")
    fn(to_dev(um), to_dev(lut), to_dev(x), out)
    w16 = o.decode(words, lut, n, L=L)
    delta = o.matvec_exact(w16, x[None])[0]
    exact = delta + init.astype(np.float64)                                # out is accumulated into (inference_t.cu:170-171)
    scale = np.linalg.norm(w16.astype(np.float64), axis=1) * np.linalg.norm(x.astype(np.float64))
    err = np.abs(out.float().cpu().numpy() - exact)
    # the product is rounded to fp16 and added to out in fp16, as the reference does: two roundings on top of the kernel's own
    tol = GEMV_HFMA2_TOL * scale + 2.0**-11 * (np.abs(delta) + np.abs(exact)) + 1e-4
    assert (err <= tol).all(), f"max err/tol {np.max(err / tol):.3f}"


def test_legacy_argument_errors():
    import rptc_kernels
    cb = torch.zeros(65536, dtype=torch.float16, device="cuda")
    comp = torch.zeros((32, 128), dtype=torch.int32, device="cuda")
    out = torch.zeros((32, 2048), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        rptc_kernels.decompress(comp.cpu(), cb, out)                     # CHECK_CUDA
    with pytest.raises(RuntimeError):
        rptc_kernels.decompress(comp.t(), cb, out)                       # CHECK_CONTIGUOUS
    with pytest.raises(RuntimeError):
        rptc_kernels.decompress(comp, cb[:100], out)                     # codebook size
    with pytest.raises(RuntimeError):
        rptc_kernels.decompress(comp, cb, out.float())                   # dtype
    with pytest.raises(RuntimeError):
        rptc_kernels.decompress_matvec_16_8_1(torch.zeros((1, 32, 64), dtype=torch.int32, device="cuda"),
                                              cb[:512], out[0], out[:, 0].contiguous())


def test_dense_probes_matvec_and_rowsum():
    # the calls of rptc_kernels/tests/test_matvec.py:18-31 and test_rowsum.py:17-30, with their rtol
    import rptc_kernels
    torch.manual_seed(42)
    m = n = 4096
    w = torch.randn((m, n), dtype=torch.float16, device="cuda")
    x = torch.randn((n,), dtype=torch.float16, device="cuda")
    out = torch.zeros((m,), dtype=torch.float16, device="cuda")
    ms = rptc_kernels.matvec(w, x, out)
    assert ms > 0
    truth = (w.float() @ x.float())
    assert (out.float() - truth).abs().max() <= 1e-3 * truth.abs().max() + 2e-2
    ms = rptc_kernels.rowsum(w, out)
    truth = w.float().sum(dim=-1)
    assert (out.float() - truth).abs().max() <= 1e-3 * truth.abs().max() + 2e-2
