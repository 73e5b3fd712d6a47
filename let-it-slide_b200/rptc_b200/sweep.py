"""Kernel sweeps over the BASELINE shapes, in the manner of the reference's print-only benchmark scripts
(rptc_kernels/tests/test_decompress.py, test_matvec.py):

    python -m rptc_b200.sweep decompress      # 4096x4096, 4096x11008, 11008x4096, 8192x28672 at K = 2, 3, 4 -> GB/s
    python -m rptc_b200.sweep gemv            # Llama-2-7B layer shapes, batch 1, 2, 4, 8 -> packed GB/s
    python -m rptc_b200.sweep gemm            # same shapes at 512 and 2048 tokens -> TFLOP/s

Every case runs over enough distinct weight buffers to exceed L2, inside one CUDA graph, timed with
CUDA events on the launching stream.  Codes are uniform random words (any bitstream is a valid
trellis path), codebooks N(0,1), activations N(0,1) fp16.
"""
from __future__ import annotations

import json
import sys

import torch

from . import CODE_HASH, CODE_LUT, LAYOUT_TILED, Format, lib, ops


def _graph_seconds(run, reps: int = 10) -> float:
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            run()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(s)
        for _ in range(reps):
            g.replay()
        b.record(s)
        b.synchronize()
    torch.cuda.current_stream().wait_stream(s)
    return a.elapsed_time(b) * 1e-3 / reps


def _codes(m: int, n: int, K: int, copies: int):
    shape = ops.codes_shape(m, n, K, LAYOUT_TILED)
    return [torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device="cuda") for _ in range(copies)]


def sweep_decompress() -> list[dict]:
    out = []
    for (m, n) in [(4096, 4096), (4096, 11008), (11008, 4096), (8192, 28672)]:
        for K in (2, 3, 4):
            fmt = Format(CODE_LUT, K, 16, 0, LAYOUT_TILED)
            lut = torch.randn(1 << 16, dtype=torch.float16, device="cuda")
            copies = max(2, int(300e6 / (m * n * 2)) + 1)
            codes = _codes(m, n, K, copies)
            dst = [torch.empty((m, n), dtype=torch.float16, device="cuda") for _ in range(copies)]

            def run():
                for c, d in zip(codes, dst):
                    ops.decompress(c, lut, m, n, fmt, out=d)

            sec = _graph_seconds(run, reps=5) / copies
            alg = m * n * K // 8 + (2 << 16) + 2 * m * n
            out.append({"kernel": "decompress", "code": "LUT L=16", "m": m, "n": n, "K": K, "us": sec * 1e6, "GB/s": alg / sec / 1e9})
            print(json.dumps(out[-1]), flush=True)
            del codes, dst
    return out


LLAMA7B = [("q/k/v/o", 4096, 4096), ("gate/up", 11008, 4096), ("down", 4096, 11008), ("qkv fused", 12288, 4096),
           ("gate-up fused", 22016, 4096)]


def sweep_gemv() -> list[dict]:
    out = []
    fmt = Format(CODE_HASH, 2, 16, 8, LAYOUT_TILED)
    lut = torch.randn(512, dtype=torch.float16, device="cuda")
    lib().rptc_set_pdl(1)
    for name, m, n in LLAMA7B:
        copies = max(2, int(300e6 / (m * n / 4)) + 1)
        codes = _codes(m, n, 2, copies)
        for batch in (1, 2, 4, 8):
            x = torch.randn((batch, n), dtype=torch.float16, device="cuda")
            acc = torch.zeros((batch, m), dtype=torch.float32, device="cuda")

            def run():
                for c in codes:
                    ops.gemv_acc(c, lut, x, acc, m, n, fmt)

            sec = _graph_seconds(run) / copies
            out.append({"kernel": "gemv", "layer": name, "m": m, "n": n, "batch": batch, "us": sec * 1e6,
                        "packed GB/s": m * n / 4 / sec / 1e9})
            print(json.dumps(out[-1]), flush=True)
        del codes
    lib().rptc_set_pdl(0)
    return out


def sweep_gemm() -> list[dict]:
    out = []
    fmt = Format(CODE_HASH, 2, 16, 8, LAYOUT_TILED)
    lut = torch.randn(512, dtype=torch.float16, device="cuda")
    for name, m, n in LLAMA7B:
        codes = _codes(m, n, 2, 1)[0]
        for tokens in (512, 2048):
            x = torch.randn((tokens, n), dtype=torch.float16, device="cuda")
            y = torch.empty((tokens, m), dtype=torch.float16, device="cuda")
            sec = _graph_seconds(lambda: ops.gemm(codes, lut, x, m, n, fmt, out=y))
            out.append({"kernel": "gemm", "layer": name, "m": m, "n": n, "tokens": tokens, "us": sec * 1e6,
                        "TFLOP/s": 2.0 * tokens * m * n / sec / 1e12})
            print(json.dumps(out[-1]), flush=True)
    return out


def main() -> None:
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which in ("decompress", "all"):
        sweep_decompress()
    if which in ("gemv", "all"):
        sweep_gemv()
    if which in ("gemm", "all"):
        sweep_gemm()
    ops.device_status()


if __name__ == "__main__":
    main()
