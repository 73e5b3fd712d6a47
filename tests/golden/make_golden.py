"""Generates tests/golden/rptc_reference_golden.npz by running the reference's OWN Python code.

    python tests/golden/make_golden.py [reference_root]     (default: $RPTC_REFERENCE_ROOT)

The reference's rptc.py, rptc_lite.py and quantize_hf.py are imported unmodified (with tests/golden/jax_shim.py
standing in for JAX, which is not installed) and their `dequantize` / `quantize` functions are run
on small seeded inputs.  The outputs are the golden vectors the CPU oracle is pinned against in
tests/test_oracle.py.  The reference checkout is only needed to REGENERATE the file; the tests read
the committed .npz.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import jax_shim  # noqa: E402


def _load(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str) -> None:
    jax_shim.install()
    rptc = _load(os.path.join(ref_root, "rptc.py"), "ref_rptc")
    lite = _load(os.path.join(ref_root, "rptc_lite.py"), "ref_rptc_lite")
    jnp = jax_shim.jnp
    rng = np.random.default_rng(42)
    out = {}

    # --- code A decode (rptc.py:74-85), L = 16 and L = 14, random symbol rows -----------------
    for L in (16, 14):
        alphabet = rng.standard_normal(1 << L).astype(np.float32)
        sym = rng.integers(0, 4, size=(3, 192)).astype(np.int32)
        dec = np.stack([np.asarray(rptc.dequantize(jnp.array(alphabet), jnp.array(s))) for s in sym])
        out[f"a{L}_alphabet"] = alphabet
        out[f"a{L}_symbols"] = sym
        out[f"a{L}_decoded"] = dec.astype(np.float32)

    # --- code A encode + decode (rptc.py:13-71) at a small state width so that it runs in seconds
    L = 8
    M = 1 << L
    alphabet = np.sort(rng.standard_normal(M)).astype(np.float32)
    alphabet = alphabet[rng.permutation(M)]
    samples = rng.standard_normal((2, 48)).astype(np.float32)
    corrections = np.eye(48, dtype=np.float32)
    qs, losses, recs = [], [], []
    for s in samples:
        q, loss = rptc.quantize(jnp.array(alphabet), jnp.array(corrections), jnp.array(s))
        qs.append(np.asarray(q))
        losses.append(float(loss))
        recs.append(np.asarray(rptc.dequantize(jnp.array(alphabet), q)))
    out["enc8_alphabet"] = alphabet
    out["enc8_samples"] = samples
    out["enc8_symbols"] = np.stack(qs).astype(np.int32)
    out["enc8_loss"] = np.array(losses, dtype=np.float64)
    out["enc8_decoded"] = np.stack(recs).astype(np.float32)

    # --- code C decode (rptc_lite.py:63-73), L=16 S=9 R=4 V=2 ----------------------------------
    L, S, R, V = 16, 9, 4, 2
    alphabet = rng.standard_normal((1 << S, V)).astype(np.float32)
    sym = rng.integers(0, 1 << R, size=(3, 96)).astype(np.int32)
    dec = np.stack([np.asarray(lite.dequantize(jnp.array(alphabet), L, S, R, jnp.array(s))) for s in sym])
    out["c_alphabet"] = alphabet
    out["c_symbols"] = sym
    out["c_decoded"] = dec.astype(np.float32)
    states = rng.integers(0, 1 << 16, size=512).astype(np.int32)
    out["c_index_states"] = states
    out["c_index"] = np.asarray(lite.index_fn(jnp.array(states), L, S)).astype(np.int32)

    # --- code C encode + decode (rptc_lite.py:19-60) at a small state width ---------------------
    L, S, R, V = 8, 5, 4, 2
    alphabet = rng.standard_normal((1 << S, V)).astype(np.float32)
    samples = rng.standard_normal((2, 24, V)).astype(np.float32)
    importance = np.ones((24, V), dtype=np.float32)
    qs, losses, recs = [], [], []
    for s in samples:
        q, loss = lite.quantize(jnp.array(alphabet), L, S, R, jnp.array(importance), jnp.array(s))
        qs.append(np.asarray(q))
        losses.append(float(loss))
        recs.append(np.asarray(lite.dequantize(jnp.array(alphabet), L, S, R, q)))
    out["encc_alphabet"] = alphabet
    out["encc_samples"] = samples
    out["encc_symbols"] = np.stack(qs).astype(np.int32)
    out["encc_loss"] = np.array(losses, dtype=np.float64)
    out["encc_decoded"] = np.stack(recs).astype(np.float32)

    # --- the HF driver's layer functions (quantize_hf.py:77-169): factorize, quantize_layer, evaluate_layer
    sys.modules["rptc"] = rptc                      # quantize_hf.py does `from rptc import quantize, dequantize`
    hf = _load(os.path.join(ref_root, "quantize_hf.py"), "ref_quantize_hf")
    W = (rng.standard_normal((24, 40)) * (1 + rng.random((24, 1))) * (0.5 + rng.random((1, 40))) + 0.3 * rng.standard_normal((24, 1))
         + 0.2 * rng.standard_normal((1, 40))).astype(np.float32)
    parts = hf.factorize(jnp.array(W))
    for name, v in zip(("biases_out", "biases_in", "scales_out", "scales_in", "normalized"), parts):
        out[f"fact_{name}"] = np.asarray(v, dtype=np.float32)
    out["fact_W"] = W
    A = rng.standard_normal((40, 64)).astype(np.float32)
    H = (A @ A.T / 64).astype(np.float32)
    recon = (W + 0.05 * rng.standard_normal(W.shape)).astype(np.float32)
    out["eval_H"], out["eval_recon"] = H, recon
    out["eval_metrics"] = np.array([float(v) for v in hf.evaluate_layer(jnp.array(H), jnp.array(W), jnp.array(recon))], dtype=np.float64)
    # quantize_layer at a small state width: 256 rows (32 banks x 1 batch x 8 rows), 16 columns, L = 8
    Wq = (rng.standard_normal((256, 16)) * (0.5 + rng.random((256, 1)))).astype(np.float32)
    Aq = rng.standard_normal((16, 32)).astype(np.float32)
    Hq = (Aq @ Aq.T / 32).astype(np.float32)
    key = 7
    out["ql_W"], out["ql_H"], out["ql_key"] = Wq, Hq, np.array(key)
    out["ql_recon"] = np.asarray(hf.quantize_layer(key, jnp.array(Hq), jnp.array(Wq), 8), dtype=np.float32)

    path = os.path.join(HERE, "rptc_reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    # the reference checkout: argument, else RPTC_REFERENCE_ROOT, else a directory `reference` beside this repository
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RPTC_REFERENCE_ROOT")
         or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
