#!/usr/bin/env python
"""Benchmark of the RPTC decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload `llama2-7b-decode-bs1`: a "step" is one decode token (batch 1 per GPU) through a Llama-2-7B-shape
network whose block linears are RPTC 2-bit (HASH code, S=8, native TILED layout, randomized-Hadamard incoherence on both
sides), random-init weights and uniform-random token ids (synthetic).  The prompt (128 tokens) is pushed through the
same decode step before timing starts.  With N > 1 every rank decodes its own sequence (replicas, weak scaling; no
data-path collective); after that measurement the same ranks run the partitioned shape, Llama-2-70B tensor-parallel over
all N GPUs, and the line carries it under the key `tp` (strong scaling: TP 2/4/8 of one model).

Beside the headline the N = 1 line carries the other kernels of the path, each timed with CUDA events on the launching
stream over buffers larger than L2: `roofline_lut` (the fused GEMV with the 65,536-entry table code), `roofline_gemm`
(the tcgen05 dequant-GEMM on the 7B layer shapes at 512 and 2048 tokens) and `roofline_decompress` (the twelve
decompression-only cases).

`--workload llama2-70b-tp` runs the partitioned shape alone.  `--workload kernels --case SPEC` times single kernels
(small enough to put under a profiler):
    gemv:MxN:bB[:hash|lut|lite]    gemm:MxN:tT[:hash|lut]    decompress:MxN:kK[:hash|lut]    all-gemv | all-gemm | all-decompress
`--plain` launches them one by one instead of replaying a CUDA graph (what a profiler should see), `--copies` sets the
number of distinct weight buffers.

`--impl reference` times the CPU restatement of the reference's decoder + matvec (oracle/, all host threads): every
step really runs all block linears of the model once.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "let-it-slide_b200"))

PROMPT = 128
METRIC = "2-bit Llama-2-7B-shape decode tok/s (bs1); dequant-GEMV GB/s vs HBM peak"
# DRAM bytes per launch over algorithmic bytes per launch of the fused GEMV, from one ncu capture of an 8192 x 8192 layer
# (16.86 MB read for 16.78 MB of packed codes + 32 KB of x and y); the traffic is proportional to the packed bytes.
GEMV_TRAFFIC_RATIO = 1.003
# ncu counters of the fused kernels on one 8192 x 8192 (GEMV: warp instructions per 128-bit unit of a 32-row block, issue
# slots used; 178 and 0.676 in the steady state of a 28672 x 8192 launch) and one 12288 x 4096 x 2048 (GEMM) launch; they
# explain the roofline fractions and are not re-measured by this script (a profiler cannot run inside a timed region).
NCU_GEMV = {"inst_per_unit": 197.0, "issue_active": 0.593, "inst_per_unit_steady": 178.0, "issue_active_steady": 0.676}
NCU_GEMM = {"tensor_active": 0.771}


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "tflops_burst": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for as long as the timed legs run.  nvidia-smi writes to a
    pseudo-terminal so that its lines arrive unbuffered (through a pipe the last second of samples stays in its stdio
    buffer and is lost when it is stopped)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines, self.fd = index, None, [], None
        self.windows: list[tuple[float, float]] = []

    def start(self):
        cmd = ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"]
        try:
            import pty
            master, slave = pty.openpty()
            self.proc = subprocess.Popen(cmd, stdout=slave, stderr=subprocess.DEVNULL, stdin=subprocess.DEVNULL, close_fds=True)
            os.close(slave)
            self.fd = master
            threading.Thread(target=self._read_fd, daemon=True).start()
        except Exception:
            try:
                self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                threading.Thread(target=self._read_pipe, daemon=True).start()
            except OSError:
                self.proc = None

    def _read_fd(self):
        buf = b""
        while True:
            try:
                chunk = os.read(self.fd, 4096)
            except OSError:
                break
            if not chunk:
                break
            buf += chunk
            *done, buf = buf.split(b"\n")
            now = time.perf_counter()
            for ln in done:
                self.lines.append((now, ln.decode(errors="replace").strip()))

    def _read_pipe(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def window(self, t0: float, t1: float) -> None:
        """Marks [t0, t1] (perf_counter) as a timed leg: its samples are the ones reported."""
        self.windows.append((t0, t1))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for when, ln in list(self.lines):
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                rows.append((when, float(f[1]), float(f[2]), float(f[3]) if f[3] not in ("[N/A]", "") else 0.0,
                             [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if any(t0 - 0.02 <= r[0] <= t1 + 0.02 for t0, t1 in self.windows)]
        where = "timed legs"
        if len(inside) < 3:           # very short legs: fall back to the samples taken while the GPU drew load power
            busy = [r for r in rows if r[3] >= 250.0]
            inside, where = (busy, "samples under load (>= 250 W)") if len(busy) >= 3 else (rows, "whole run")
        sm = [r[1] for r in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max((r[2] for r in rows), default=None),
                "reasons": sorted({n for r in inside for n in r[4]}), "samples": len(sm), "window": where,
                "power_w_max": max((r[3] for r in inside), default=None)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle's C restatement of decode + matvec over every block linear of the model
# ------------------------------------------------------------------------------------------------
class CpuModel:
    """All block linears of the model as packed codes in host memory (distinct buffers per layer, seeded), and one decode
    token's worth of work on them: decode + fp32 matvec of every linear through the C oracle, all host threads."""

    def __init__(self, cfg_dims: dict, max_layers: int | None = None):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import numpy as np

        import c_oracle
        self.np, self.c = np, c_oracle
        # all the host cores this process may run on, whatever a launcher exported as OMP_NUM_THREADS for its children
        c_oracle.set_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
        hidden, ffn, self.layers = cfg_dims["hidden"], cfg_dims["ffn"], cfg_dims["layers"]
        q, kv = cfg_dims["heads"] * 128, cfg_dims["kv_heads"] * 128
        shapes = [(q + 2 * kv, hidden), (hidden, q), (2 * ffn, hidden), (hidden, ffn)]
        self.built = self.layers if max_layers is None else min(self.layers, max_layers)
        rng = np.random.default_rng(42)
        self.lut = rng.standard_normal(512).astype(np.float16)
        self.mats = []
        for _ in range(self.built):
            for (m, n) in shapes:
                self.mats.append((rng.integers(0, 2**32, (m, n // 16), dtype=np.uint32), rng.standard_normal((1, n)).astype(np.float16), m, n))
        self.weights_per_token = sum(m * n for _, _, m, n in self.mats) * self.layers // self.built

    def token(self) -> float:
        """Seconds for one decode token's block linears (scaled when only some of the layers were built)."""
        t0 = time.perf_counter()
        for words, x, m, n in self.mats:
            self.c.gemv(words, self.lut, x, m, n, code=1, K=2, L=16, S=8, layout=0)
        return (time.perf_counter() - t0) * self.layers / self.built

    def describe(self, tokens: int) -> str:
        part = "" if self.built == self.layers else f" ({self.built} of {self.layers} layers timed, scaled)"
        return (f"{tokens} decode tokens, each the decode + fp32 matvec of all {self.layers * 4} RPTC block linears "
                f"({self.weights_per_token / 1e9:.2f}G weights){part}; norms, attention and the output head not included")


def bytes_per_token(cfg_dims: dict, context: int, tp_world: int = 1) -> dict:
    """Bytes one decode token streams: packed block linears (2 bits per weight), the fp16 output head, the KV rows read."""
    hidden, ffn, layers = cfg_dims["hidden"], cfg_dims["ffn"], cfg_dims["layers"]
    q, kv = cfg_dims["heads"] * 128, cfg_dims["kv_heads"] * 128
    weights = layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * ffn)
    return {"packed": weights * 2 // 8 // tp_world, "head": 32000 * hidden * 2, "kv": 2 * layers * context * (kv // tp_world) * 2}


def config_of(args, cfg_dims: dict, world: int, tp: bool) -> dict:
    """The workload description both arms print (the reference arm runs the same codes and shapes on the host)."""
    ctx = args.prompt + args.warmup + args.steps // 2
    return {"workload": args.workload, "code": "HASH S=8 K=2 L=16", "layout": "TILED", "incoherence": "RHT both sides",
            "prompt": args.prompt, "batch_per_gpu": 1, "allreduce": (args.allreduce if tp else None),
            "parallelism": (f"tp{world}" if tp else ("replicas" if world > 1 else "single")),
            "l2": "weights 1.6 GB per token exceed L2", "bytes_per_token": bytes_per_token(cfg_dims, ctx, world if tp else 1)}


def run_reference(args, cfg_dims: dict) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    big = cfg_dims["layers"] * cfg_dims["hidden"] > 200000          # the 70B shape: 17 GB of codes, a sample of its layers
    cpu = CpuModel(cfg_dims, max_layers=8 if big else None)
    for _ in range(args.warmup):
        cpu.token()
    t0 = time.perf_counter()
    times = [cpu.token() for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    sec = statistics.mean(times)
    val = 1.0 / sec
    out = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f16", "data": "synthetic",
           "config": config_of(args, cfg_dims, int(os.environ.get("WORLD_SIZE", "1")), args.workload.endswith("-tp")),
           "timed_wall_s": wall,
           "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cpu.c.threads(), "kind": "port", "sample": cpu.describe(args.steps)},
           "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------------
# GPU arm: timing helpers
# ------------------------------------------------------------------------------------------------
def graph_seconds(torch, run, reps: int = 10, plain: bool = False, sampler: ClockSampler | None = None) -> float:
    """Seconds per call of `run` (a fixed sequence of launches): replayed as one CUDA graph (or launched as it is with
    `plain`), CUDA events on the launching stream, three untimed runs first."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        if plain:
            go = run
        else:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                run()
            g.replay()
            go = g.replay
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        a.record(s)
        for _ in range(reps):
            go()
        b.record(s)
        b.synchronize()
        if sampler is not None:
            sampler.window(t0, time.perf_counter())
    torch.cuda.current_stream().wait_stream(s)
    return a.elapsed_time(b) * 1e-3 / reps


def gemv_roofline(torch, linears, kernel: str, sampler=None, reps: int = 5) -> dict:
    """Times the fused dequant-GEMV alone over all of `linears` (distinct weight buffers, far more than L2) inside one
    CUDA graph, launched the way the decode step launches them (programmatic dependent launch)."""
    from rptc_b200 import lib
    dev = linears[0].codes.device
    xs = {l.in_features: torch.randn((1, l.in_features), dtype=torch.float16, device=dev) for l in linears}
    accs = {l.out_features: torch.zeros((1, l.out_features), dtype=torch.float32, device=dev) for l in linears}

    def run():
        for l in linears:
            l.matvec_acc(xs[l.in_features], accs[l.out_features])

    lib().rptc_set_pdl(1)
    try:
        sec = graph_seconds(torch, run, reps, sampler=sampler)
    finally:
        lib().rptc_set_pdl(0)
    K = linears[0].fmt.K
    alg = sum(l.in_features * l.out_features * K // 8 + 2 * l.in_features + 4 * l.out_features + 2 * l.lut.numel() for l in linears)
    packed = sum(l.in_features * l.out_features * K // 8 for l in linears)
    peaks = measured_peaks()
    n = len(linears)
    achieved = alg / sec / 1e9
    return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth", "traffic": alg / n * GEMV_TRAFFIC_RATIO,
            "algorithmic_bytes_per_launch": alg / n, "launch_us": sec / n * 1e6, "launches_timed": n * reps,
            "packed_stream_gbs": packed / sec / 1e9, "frac_of_8000": packed / sec / 1e9 / 8000.0}


def issue_bound(roof: dict, sm_mhz: float | None, sms: int = 148) -> None:
    """What the instruction stream permits: SMs x 4 warp instructions per clock x clock / instructions per 128-bit unit of
    32 rows x 512 bytes per unit (2048 weights at 2 bits): at every issue slot used (`issue_bound_gbs`), at the measured
    utilisation (`issue_bound_gbs_at_measured_utilisation`), and for the 136 instructions per unit that the code's
    definition demands (32 lookups, 32 hashes, 32 address splices, 32 window shifts, 8 tensor-core instructions).
    Counters from the ncu captures named above."""
    f = (sm_mhz or 1965.0) * 1e6
    roof["inst_per_unit"] = NCU_GEMV["inst_per_unit"]
    roof["issue_active"] = NCU_GEMV["issue_active"]
    roof["issue_bound_gbs"] = sms * 4 * f / NCU_GEMV["inst_per_unit"] * 512 / 1e9
    roof["issue_bound_gbs_at_measured_utilisation"] = sms * 4 * f * NCU_GEMV["issue_active_steady"] / NCU_GEMV["inst_per_unit_steady"] * 512 / 1e9
    roof["issue_bound_gbs_essential_136_inst"] = sms * 4 * f / 136.0 * 512 / 1e9


LLAMA7B_LAYERS = [("q/k/v/o", 4096, 4096), ("gate/up", 11008, 4096), ("down", 4096, 11008), ("qkv fused", 12288, 4096),
                  ("gate-up fused", 22016, 4096)]
DECOMPRESS_SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096), (8192, 28672)]


def _fmt(kind: str, K: int = 2):
    from rptc_b200 import CODE_HASH, CODE_LITE, CODE_LUT, LAYOUT_TILED, Format
    if kind == "lut":
        return Format(CODE_LUT, K, 16, 0, LAYOUT_TILED)
    if kind == "lite":
        return Format(CODE_LITE, K, 16, 9, LAYOUT_TILED)
    return Format(CODE_HASH, 2, 16, 8, LAYOUT_TILED)


def _codes(torch, ops, m, n, K, copies):
    from rptc_b200 import LAYOUT_TILED
    shape = ops.codes_shape(m, n, K, LAYOUT_TILED)
    return [torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device="cuda") for _ in range(copies)]


def time_gemv(torch, m, n, batch, kind="hash", copies=None, plain=False, reps=10, sampler=None) -> dict:
    from rptc_b200 import lib, ops
    fmt = _fmt(kind)
    lut = torch.randn(fmt.lut_numel(), dtype=torch.float16, device="cuda")
    copies = copies or max(2, int(300e6 / (m * n / 4)) + 1)
    codes = _codes(torch, ops, m, n, fmt.K, copies)
    x = torch.randn((batch, n), dtype=torch.float16, device="cuda")
    acc = torch.zeros((batch, m), dtype=torch.float32, device="cuda")

    def run():
        for c in codes:
            ops.gemv_acc(c, lut, x, acc, m, n, fmt)

    lib().rptc_set_pdl(1)
    try:
        sec = graph_seconds(torch, run, reps, plain, sampler) / copies
    finally:
        lib().rptc_set_pdl(0)
    gbs = m * n * fmt.K / 8 / sec / 1e9
    return {"kernel": "gemv", "code": kind, "m": m, "n": n, "batch": batch, "us": sec * 1e6, "packed_gbs": gbs,
            "frac": gbs / measured_peaks()["hbm_gbs"], "copies": copies}


def time_gemm(torch, m, n, tokens, kind="hash", plain=False, reps=10, sampler=None, unfused=False) -> dict:
    from rptc_b200 import ops
    fmt = _fmt(kind)
    lut = torch.randn(fmt.lut_numel(), dtype=torch.float16, device="cuda")
    codes = _codes(torch, ops, m, n, fmt.K, 1)[0]
    x = torch.randn((tokens, n), dtype=torch.float16, device="cuda")
    y = torch.empty((tokens, m), dtype=torch.float16, device="cuda")
    sec = graph_seconds(torch, lambda: ops.gemm(codes, lut, x, m, n, fmt, out=y), reps, plain, sampler)
    tf = 2.0 * tokens * m * n / sec / 1e12
    out = {"kernel": "gemm", "code": kind, "m": m, "n": n, "tokens": tokens, "us": sec * 1e6, "tflops": tf,
           "frac": tf / measured_peaks()["tflops"]}
    if unfused:
        # the two-step alternative the fused kernel replaces: decompress to dense fp16, then a library GEMM (cuBLAS)
        dense = torch.empty((m, n), dtype=torch.float16, device="cuda")

        def two_step():
            ops.decompress(codes, lut, m, n, fmt, out=dense)
            torch.matmul(x, dense.t(), out=y)

        out["decompress_plus_cublas_us"] = graph_seconds(torch, two_step, reps, plain) * 1e6
        out["cublas_alone_us"] = graph_seconds(torch, lambda: torch.matmul(x, dense.t(), out=y), reps, plain) * 1e6
    return out


def time_decompress(torch, m, n, K, kind="lut", copies=None, plain=False, reps=5, sampler=None) -> dict:
    from rptc_b200 import ops
    fmt = _fmt(kind, K)
    lut = torch.randn(fmt.lut_numel(), dtype=torch.float16, device="cuda")
    copies = copies or max(2, int(300e6 / (m * n * 2)) + 1)
    codes = _codes(torch, ops, m, n, K, copies)
    dst = [torch.empty((m, n), dtype=torch.float16, device="cuda") for _ in range(copies)]

    def run():
        for c, d in zip(codes, dst):
            ops.decompress(c, lut, m, n, fmt, out=d)

    sec = graph_seconds(torch, run, reps, plain, sampler) / copies
    alg = m * n * K // 8 + 2 * fmt.lut_numel() + 2 * m * n
    gbs = alg / sec / 1e9
    return {"kernel": "decompress", "code": kind, "m": m, "n": n, "K": K, "us": sec * 1e6, "gbs": gbs,
            "frac": gbs / measured_peaks()["hbm_gbs"], "algorithmic_bytes": alg}


def run_kernels(args) -> None:
    import torch
    from rptc_b200 import ops
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    case = args.case or "all-gemv"

    def dims(s):
        m, n = s.lower().split("x")
        return int(m), int(n)

    if case.startswith("all-"):
        which = case[4:]
        if which == "gemv":
            for kind in ("hash", "lut"):
                for _, m, n in LLAMA7B_LAYERS + [("70B gate-up", 28672, 8192), ("70B down", 8192, 28672)]:
                    for b in (1, 2, 4, 8):
                        print(json.dumps(time_gemv(torch, m, n, b, kind, plain=args.plain)), flush=True)
        elif which == "gemm":
            for _, m, n in LLAMA7B_LAYERS:
                for t in (512, 2048):
                    print(json.dumps(time_gemm(torch, m, n, t, plain=args.plain, unfused=not args.plain)), flush=True)
        elif which == "decompress":
            for m, n in DECOMPRESS_SHAPES:
                for K in (2, 3, 4):
                    print(json.dumps(time_decompress(torch, m, n, K, plain=args.plain)), flush=True)
        else:
            raise SystemExit(f"unknown case {case}")
    else:
        f = case.split(":")
        m, n = dims(f[1])
        kind = f[3] if len(f) > 3 else None
        if f[0] == "gemv":
            out = time_gemv(torch, m, n, int(f[2].lstrip("b")), kind or "hash", args.copies, args.plain, args.reps)
        elif f[0] == "gemm":
            out = time_gemm(torch, m, n, int(f[2].lstrip("t")), kind or "hash", args.plain, args.reps, unfused=not args.plain)
        elif f[0] == "decompress":
            out = time_decompress(torch, m, n, int(f[2].lstrip("k")), kind or "lut", args.copies, args.plain, args.reps)
        else:
            raise SystemExit(f"unknown case {case}")
        print(json.dumps(out), flush=True)
    torch.cuda.synchronize()
    ops.device_status()


# ------------------------------------------------------------------------------------------------
# GPU arm: the decode workloads
# ------------------------------------------------------------------------------------------------
def decode_leg(args, torch, dist, cfg_kw, tp: bool, allreduce: str, world: int, rank: int, sampler, prompt_len: int, rows: int = 1):
    """Builds the model, pushes the prompt through the decode step, then times `steps` tokens twice: token feedback on the
    device (CUDA events) and host in the loop every step (wall clock).  Returns (model, device ms, e2e ms, h2d, d2h)."""
    from rptc_b200 import ops
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(max_pos=prompt_len + max(3, args.warmup) + 2 * args.steps + 8, **cfg_kw)
    if tp:
        model = RPTCLlama(cfg, rows=rows, seed=0, tp_world=world, tp_rank=rank, peer_allreduce=allreduce == "peer")
    else:
        model = RPTCLlama(cfg, rows=rows, seed=rank)
    g = torch.Generator(device="cuda").manual_seed(42 + (0 if tp else rank))
    prompt = torch.randint(0, cfg.vocab, (prompt_len, rows), device="cuda", generator=g, dtype=torch.int32)
    model.reset()
    model.capture(pdl=True)
    for t in range(prompt_len):                            # the prompt goes through the decode step, token by token
        model.ids.copy_(prompt[t])
        model.step()
    for _ in range(max(3, args.warmup)):
        model.step()
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident decode: token feedback stays on the GPU ----
    barrier()
    pos_timed = model.pos.clone()          # both timed legs decode the same positions (same attention work)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    a.record()
    for _ in range(args.steps):
        model.step()
    b.record()
    b.synchronize()
    sampler.window(w0, time.perf_counter())
    barrier()
    ms = a.elapsed_time(b)
    # ---- end to end: host token in, host token out, every step ----
    # Single GPU / replicas: the mailbox loop of rptc_b200.llama.HostTokenLoop -- the host posts each step's token id
    # in pinned memory (8 bytes, read over PCIe by the step's first kernel) and polls the id the step's last kernel
    # writes back (8 bytes), keeping one graph launch queued ahead.  Tensor parallel: the step's first kernel reads a
    # pinned int32, the last writes a pinned int64, and the host synchronises the stream every step.
    first = model.ids.tolist()
    torch.cuda.synchronize()
    model.pos.copy_(pos_timed - 3)         # three untimed steps, then the positions of the device-resident leg
    model.sync_positions()
    if not tp:
        loop = model.host_loop()
        first = loop.run(first, 3)[-1]
        h2d, d2h = 8 * rows, 8 * rows
        barrier()
        t0 = time.perf_counter()
        loop.run(first, args.steps)
        torch.cuda.synchronize()
    else:
        host_in = torch.zeros(rows, dtype=torch.int32).pin_memory()
        host_out = torch.zeros(rows, dtype=torch.int64).pin_memory()
        host_in.copy_(torch.tensor(first, dtype=torch.int32))
        model.bind_host_io(host_in, host_out)
        model.capture(pdl=True)
        h2d, d2h = 4 * rows, 8 * rows
        for _ in range(3):
            model.step()
            torch.cuda.current_stream().synchronize()
            host_in.copy_(host_out.to(torch.int32))
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.step()
            torch.cuda.current_stream().synchronize()
            host_in.copy_(host_out.to(torch.int32))
    t1 = time.perf_counter()
    sampler.window(t0, t1)
    barrier()
    ops.device_status()
    t = torch.tensor([ms, (t1 - t0) * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    return model, ms, e2e_ms, h2d, d2h


def allreduce_us(torch, dist, model, world: int, reps: int = 3) -> float | None:
    """Microseconds per all-reduce of the tensor-parallel step, measured on a graph of nothing but the step's 2 x layers
    all-reduces of the row-parallel outputs (every rank runs the same count, max over ranks)."""
    if model.peer is None:
        return None
    lin = model.blocks[0].o
    n = 2 * len(model.blocks)

    def run():
        for _ in range(n):
            model.peer.finish(lin, model.acc_h, model.h)

    from rptc_b200 import lib
    lib().rptc_set_pdl(1)
    try:
        torch.cuda.synchronize()
        dist.barrier()
        sec = graph_seconds(torch, run, reps)
    finally:
        lib().rptc_set_pdl(0)
    t = torch.tensor([sec], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / n * 1e6


def kernel_timeline(torch, model, steps: int = 4, dist=None) -> dict:
    """Where a decode step's time goes, kernel by kernel: the captured step is replayed under torch.profiler (CUPTI kernel
    records) and every kernel is charged the time between the end of the kernel before it and its own end -- the chain is
    serial, so these add up to the step.  Diagnostic only (`--timeline`): run after the timed legs, never inside them."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    if model.mailbox is not None or model.host_ids is not None:
        # the end-to-end leg left the step waiting for tokens from the host: back to device-resident feedback
        model.mailbox = None
        model.bind_host_io(None, None)
        model.capture(pdl=True)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        if dist is not None:
            # the profiler starts up seconds apart on different ranks, longer than the all-reduce kernel waits for a peer
            dist.barrier()
            torch.cuda.synchronize()
        for _ in range(steps):
            model.step()
        torch.cuda.synchronize()
    from rptc_b200 import ops
    ops.device_status()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end > e.time_range.start
          and "nccl" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    own, crit, cnt = collections.defaultdict(float), collections.defaultdict(float), collections.Counter()
    last_end = None
    for e in ev:
        name = e.name.split("(")[0].replace("void ", "").replace("rptc::", "")
        own[name] += e.time_range.end - e.time_range.start
        cnt[name] += 1
        if last_end is not None:
            crit[name] += max(0.0, e.time_range.end - last_end)
        last_end = max(last_end or 0, e.time_range.end)
    total = sum(crit.values())
    rows = [{"kernel": k, "launches_per_step": cnt[k] / steps, "own_us": own[k] / cnt[k], "critical_us": crit[k] / cnt[k],
             "critical_us_per_step": crit[k] / steps, "share": crit[k] / total} for k in sorted(crit, key=lambda k: -crit[k])]
    return {"us_per_step": total / steps, "kernels": rows}


def close_model(torch, dist, model, world: int) -> None:
    model.graph = None              # graphs that captured collectives must be gone before their communicator is torn down
    torch.cuda.synchronize()
    if getattr(model, "peer", None) is not None:
        model.peer.close()
        model.peer = None
    if world > 1:
        dist.barrier()


def tp_record(args, torch, dist, world, rank, sampler, allreduce: str, rows: int = 1) -> dict | None:
    """The partitioned shape on all ranks: Llama-2-70B, column/row splits, one all-reduce after o and down; `rows`
    sequences decode together (batch 1 and 16)."""
    cfg_kw, _ = WORKLOADS["llama2-70b-tp"]
    model, ms, e2e_ms, h2d, d2h = decode_leg(args, torch, dist, cfg_kw, True, allreduce, world, rank, sampler, min(args.prompt, 32), rows)
    ar_us = allreduce_us(torch, dist, model, world) if world > 1 else None
    bt = model.bytes_per_token(min(args.prompt, 32) + args.warmup + args.steps // 2)
    step_s = ms / args.steps * 1e-3
    peaks = measured_peaks()
    rec = {"workload": "llama2-70b-tp", "batch": rows, "tok_s": rows * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
           "allreduce": allreduce, "parallelism": f"tp{world}", "launches_per_step": model.launches_per_step, "us_per_allreduce": ar_us,
           "allreduces_per_step": 2 * len(model.blocks), "packed_gb_per_gpu": bt["packed"] / 1e9,
           "e2e_tok_s": rows * args.steps / (e2e_ms * 1e-3), "scaling": "strong",
           "roofline": {"bound": "hbm", "achieved": bt["packed"] / step_s / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": bt["packed"] / step_s / 1e9 / peaks["hbm_gbs"], "what": "packed codes per GPU per token / step time"}}
    if args.timeline:
        if world > 1:
            dist.barrier()
        rec["timeline"] = kernel_timeline(torch, model, dist=dist if world > 1 else None)
    close_model(torch, dist, model, world)
    del model
    torch.cuda.empty_cache()
    return rec if rank == 0 else None


def run_ours(args, cfg_kw: dict, cfg_dims: dict) -> None:
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from rptc_b200 import ops
    from rptc_b200.linear import RPTCLinear

    tp = args.workload.endswith("-tp")
    sampler = ClockSampler(local)
    sampler.start()
    model, ms, e2e_ms, h2d, d2h = decode_leg(args, torch, dist, cfg_kw, tp, args.allreduce, world, rank, sampler, args.prompt)
    out = None
    if rank == 0:
        linears = [l for b in model.blocks for l in b.linears()]
        roof = gemv_roofline(torch, linears, "gemv_rows_kernel<HASH,K=2,batch=1>", sampler)
        bt = bytes_per_token(cfg_dims, args.prompt + args.warmup + args.steps // 2, world if tp else 1)
        seqs = 1 if tp else world
        out = {"metric": METRIC if not tp else "2-bit Llama-2-70B-shape tensor-parallel decode tok/s (bs1)",
               "value": seqs * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if tp else "weak",
               "vs_baseline": None, "dtype": "f16", "data": "synthetic",
               "config": config_of(args, cfg_dims, world, tp),
               "e2e": {"value": seqs * args.steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               "gpu_launches": model.launches_per_step * args.steps, "roofline": roof,
               "token_stream_gbs": (bt["packed"] + bt["head"] + bt["kv"]) / (ms / args.steps * 1e-3) / 1e9}
    if args.timeline and (tp or rank == 0):          # tensor parallel: every rank must run the steps
        if tp and world > 1:
            dist.barrier()
        tl = kernel_timeline(torch, model, dist=dist if (tp and world > 1) else None)
        if rank == 0:
            out["timeline"] = tl
    launches_per_step = model.launches_per_step
    close_model(torch, dist, model, world)
    del model
    torch.cuda.empty_cache()

    if world == 1 and not tp and args.extras and rank == 0:
        # ---- the other kernels of the path (N = 1 only) ----
        peaks = measured_peaks()
        fmt_lut = _fmt("lut")
        shapes = [(4096, 12288), (4096, 4096), (4096, 22016), (11008, 4096)]           # (in, out) of a 7B block's four linears
        lut_linears = [RPTCLinear.random(i, o, fmt_lut, 0.02, 1000 + 4 * layer + k, "cuda", incoherent=False)
                       for layer in range(32) for k, (i, o) in enumerate(shapes)]
        out["roofline_lut"] = gemv_roofline(torch, lut_linears, "gemv_rows_kernel<LUT L=16,K=2,batch=1>", sampler)
        del lut_linears
        torch.cuda.empty_cache()
        gemm = [time_gemm(torch, m, n, t, sampler=sampler, unfused=True) | {"layer": name} for name, m, n in LLAMA7B_LAYERS for t in (512, 2048)]
        big = next(c for c in gemm if c["m"] == 12288 and c["tokens"] == 2048)
        out["roofline_gemm"] = {"bound": "tensor", "kernel": "gemm_kernel<HASH,K=2> (tcgen05, TMEM accumulators)", "achieved": big["tflops"],
                                "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": big["frac"], "case": "12288x4096, 2048 tokens",
                                "peak_source": f"{peaks['source']} sustained bf16 cuBLAS", "flops": "2*T*m*n", "traffic": None,
                                "tensor_active": NCU_GEMM["tensor_active"], "cases": gemm}
        dec = [time_decompress(torch, m, n, K, sampler=sampler) for m, n in DECOMPRESS_SHAPES for K in (2, 3, 4)]
        worst, best = min(dec, key=lambda c: c["frac"]), max(dec, key=lambda c: c["frac"])
        out["roofline_decompress"] = {"bound": "hbm", "kernel": "decompress_kernel<LUT L=16>", "unit": "GB/s", "peak": peaks["hbm_gbs"],
                                      "achieved": statistics.mean(c["gbs"] for c in dec), "frac": statistics.mean(c["frac"] for c in dec),
                                      "frac_min": worst["frac"], "frac_max": best["frac"], "bytes": "m*n*K/8 + 2^L*2 + 2*m*n",
                                      "peak_source": f"{peaks['source']} copy bandwidth", "cases": dec}
        ops.device_status()
        # decode batch 16 of the same 7B shape (sixteen sequences step together)
        m16, ms16, e2e16, _, _ = decode_leg(args, torch, dist, cfg_kw, False, args.allreduce, 1, 0, sampler, min(args.prompt, 32), rows=16)
        out["decode_bs16"] = {"tok_s": 16 * args.steps / (ms16 * 1e-3), "ms_per_step": ms16 / args.steps,
                              "e2e_tok_s": 16 * args.steps / (e2e16 * 1e-3), "launches_per_step": m16.launches_per_step}
        close_model(torch, dist, m16, 1)
        del m16
        torch.cuda.empty_cache()

    if world > 1 and not tp and args.extras:
        # ---- the partitioned shape on the same ranks ----
        rec = tp_record(args, torch, dist, world, rank, sampler, "peer")
        if rank == 0:
            out["tp"] = rec
        rec = tp_record(args, torch, dist, world, rank, sampler, "peer", rows=16)
        if rank == 0:
            out["tp_bs16"] = rec
        if args.tp_nccl:
            rec = tp_record(args, torch, dist, world, rank, sampler, "nccl")
            if rank == 0:
                out["tp_nccl"] = rec

    clocks = sampler.stop()
    if rank == 0:
        out["clocks"] = clocks
        issue_bound(out["roofline"], clocks.get("sm_mhz"))
        if world == 1:
            cpu = CpuModel(cfg_dims, max_layers=None if not tp else 4)
            cpu.token()
            secs = [cpu.token() for _ in range(3)]
            out["cpu_baseline"] = {"value": 1.0 / statistics.mean(secs), "unit": "tok/s", "cores": cpu.c.threads(), "kind": "port",
                                   "sample": cpu.describe(3)}
        else:
            out["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": "timed at N = 1 only"}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


WORKLOADS = {
    "llama2-7b-decode-bs1": (dict(), dict(hidden=4096, ffn=11008, layers=32, heads=32, kv_heads=32)),
    # the partitioned shape: tensor-parallel over all ranks (strong scaling), one all-reduce after o and down (--allreduce)
    "llama2-70b-tp": (dict(hidden=8192, layers=80, heads=64, kv_heads=8, ffn=28672),
                      dict(hidden=8192, ffn=28672, layers=80, heads=64, kv_heads=8)),
    "kernels": (None, None),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama2-7b-decode-bs1", choices=list(WORKLOADS))
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="tensor-parallel workloads: fused peer-memory all-reduce kernel, or NCCL")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt tokens pushed through the decode step before timing")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="headline only: skip the other kernels' rooflines (N = 1) and the tensor-parallel leg (N > 1)")
    ap.add_argument("--tp-nccl", action="store_true", help="N > 1: also run the tensor-parallel leg with NCCL all-reduces")
    ap.add_argument("--timeline", action="store_true", help="add each decode leg's per-kernel critical-path times (torch.profiler)")
    ap.add_argument("--case", default=None, help="--workload kernels: which kernel and shape (see the module docstring)")
    ap.add_argument("--plain", action="store_true", help="--workload kernels: plain launches instead of a CUDA graph")
    ap.add_argument("--copies", type=int, default=None, help="--workload kernels: distinct weight buffers per case")
    ap.add_argument("--reps", type=int, default=10, help="--workload kernels: timed repetitions")
    args = ap.parse_args()
    if args.workload == "kernels":
        if args.impl == "reference":
            raise SystemExit("the reference arm runs the decode workloads")
        return run_kernels(args)
    cfg_kw, cfg_dims = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg_dims)
    else:
        run_ours(args, cfg_kw, cfg_dims)


if __name__ == "__main__":
    main()
