"""Runs ONE entry point of the compiled, unmodified reference extension (oracle/_ref, built by
oracle/build_ref.sh) on seeded inputs and saves inputs + output to an .npz.

It runs as a child process of the GPU tests because the reference calls exit() on any CUDA error
(inference.cu:32-39), which must not take the test session down with it.

    python tests/ref_runner.py <decompress|matvec_16_8_1|matvec_16_6_1|matvec_t_16> <out.npz> <m> <n> <seed> [words.npy]

With a sixth argument the stream words ([m, n/16] uint32, row-major) are read from that file instead of being drawn.
Exit codes: 0 done, 3 the reference extension is not built, 4 unknown entry point.
"""
import glob
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_reference():
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", "rptc_kernels_reference*.so"))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location("rptc_kernels_reference", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    which, path, m, n, seed = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5])
    ref = load_reference()
    if ref is None:
        sys.exit(3)
    rng = np.random.default_rng(seed)
    words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)      # row-major stream words
    if len(sys.argv) > 6:
        words = np.load(sys.argv[6]).astype(np.uint32)
        assert words.shape == (m, n // 16)
    x = rng.standard_normal(n).astype(np.float16)
    res = {"words": words, "x": x}
    dev = "cuda"
    if which == "decompress":
        lut = rng.standard_normal(1 << 16).astype(np.float16)
        out = torch.zeros((m, n), dtype=torch.float16, device=dev)
        ref.decompress(torch.from_numpy(words.view(np.int32)).to(dev), torch.from_numpy(lut).to(dev), out)
    elif which.startswith("matvec_16_"):
        S = int(which.split("_")[2])
        lut = rng.standard_normal(2 << S).astype(np.float16)
        chunked = np.ascontiguousarray(words.reshape(m, n // 2048, 128).transpose(1, 0, 2))
        out = torch.zeros((m,), dtype=torch.float16, device=dev)
        fn = getattr(ref, f"decompress_matvec_16_{S}_1")
        fn(torch.from_numpy(chunked.view(np.int32)).to(dev), torch.from_numpy(lut).to(dev), torch.from_numpy(x).to(dev), out)
    elif which == "matvec_t_16":
        lut = rng.standard_normal(1 << 16).astype(np.float16)
        um = np.ascontiguousarray(words.reshape(m, n // 64, 4).transpose(1, 0, 2))
        init = rng.standard_normal(m).astype(np.float16)
        res["init"] = init
        out = torch.from_numpy(init.copy()).to(dev)
        ref.decompress_matvec_t_16(torch.from_numpy(um.view(np.int32)).to(dev), torch.from_numpy(lut).to(dev),
                                   torch.from_numpy(x).to(dev), out)
    else:
        sys.exit(4)
    torch.cuda.synchronize()
    res["lut"] = lut
    res["out"] = out.cpu().numpy()
    np.savez(path, **res)


if __name__ == "__main__":
    main()
