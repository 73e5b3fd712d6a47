#!/usr/bin/env python
"""Benchmark of the RPTC decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one decode token (batch 1 per GPU) through a Llama-2-7B-shape network whose block
linears are RPTC 2-bit (HASH code, S=8, native TILED layout, randomized-Hadamard incoherence on
both sides), random-init weights and uniform-random token ids (synthetic).  The
prompt (128 tokens) is pushed through the same decode step before timing starts.  With N > 1 every
rank decodes its own sequence (replicas, weak scaling; no data-path collective): only the 70B shape
is partitioned, `--workload llama2-70b-tp`.

`--impl reference` times the CPU restatement of the reference's decoder + matvec (oracle/, all
host threads) on a bounded sample of the same workload.
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
# dram bytes per launch / algorithmic bytes per launch of the fused GEMV, from the ncu capture summarised in
# profiles/gemv_hash_k2_8192x8192.md (16.86 MB read for 16.78 MB packed + 32 KB of x and y)
GEMV_TRAFFIC_RATIO = 1.003


def measured_hbm_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle's C restatement of decode + matvec, on one decoder block's linears
# ------------------------------------------------------------------------------------------------
def cpu_block_seconds(cfg_dims: dict, reps: int) -> tuple[float, int, str]:
    """Seconds per decode token extrapolated from timing one block's four linears on the host."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np

    import c_oracle
    # all the host cores this process may run on, whatever a launcher exported as OMP_NUM_THREADS for its children
    c_oracle.set_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    hidden, ffn, layers = cfg_dims["hidden"], cfg_dims["ffn"], cfg_dims["layers"]
    q = cfg_dims["heads"] * 128
    kv = cfg_dims["kv_heads"] * 128
    shapes = [(q + 2 * kv, hidden), (hidden, q), (2 * ffn, hidden), (hidden, ffn)]
    rng = np.random.default_rng(42)
    lut = rng.standard_normal(512).astype(np.float16)
    mats = []
    for (m, n) in shapes:
        words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)
        x = rng.standard_normal((1, n)).astype(np.float16)
        mats.append((words, x, m, n))
    best = float("inf")
    for _ in range(max(1, reps)):
        t0 = time.perf_counter()
        for words, x, m, n in mats:
            c_oracle.gemv(words, lut, x, m, n, code=1, K=2, L=16, S=8, layout=0)
        best = min(best, time.perf_counter() - t0)
    weights = sum(m * n for _, _, m, n in mats)
    sample = (f"decode+matvec (fp32 accumulate) of one of {layers} decoder blocks' four RPTC linears "
              f"({weights / 1e6:.0f}M weights), best of {max(1, reps)}, scaled by {layers}; norms/attention/head not included")
    return best * layers, c_oracle.threads(), sample


def run_reference(args, cfg_dims: dict) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_block_seconds(cfg_dims, 1)
    times = [cpu_block_seconds(cfg_dims, 1) for _ in range(max(1, min(args.steps, 8)))]
    sec = statistics.mean(t[0] for t in times)
    cores, sample = times[0][1], times[0][2]
    val = 1.0 / sec
    out = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f16", "data": "synthetic", "config": {"workload": args.workload, "prompt": PROMPT, "batch_per_gpu": 1},
           "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def gemv_roofline(model, torch, reps: int = 5) -> dict:
    """Times the fused dequant-GEMV alone over all block linears of the model (distinct weight buffers,
    1.6 GB > L2) inside one CUDA graph, with events on the launching stream."""
    from rptc_b200 import lib
    linears = [l for b in model.blocks for l in b.linears()]
    xs = {l.in_features: torch.randn((1, l.in_features), dtype=torch.float16, device=model.device) for l in linears}
    accs = {l.out_features: torch.zeros((1, l.out_features), dtype=torch.float32, device=model.device) for l in linears}

    def run():
        for l in linears:
            l.matvec_acc(xs[l.in_features], accs[l.out_features])

    lib().rptc_set_pdl(1)      # launched the way the decode step launches it
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
    lib().rptc_set_pdl(0)
    sec = a.elapsed_time(b) * 1e-3 / reps
    K = model.fmt.K
    alg = sum(l.in_features * l.out_features * K // 8 + 2 * l.in_features + 4 * l.out_features + 2 * l.lut.numel() for l in linears)
    packed = sum(l.in_features * l.out_features * K // 8 for l in linears)
    peak, src = measured_hbm_peak()
    n = len(linears)
    achieved = alg / sec / 1e9
    return {"bound": "hbm", "kernel": "gemv_pair_kernel<HASH,K=2,batch=1>", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": f"{src} copy bandwidth", "traffic": alg / n * GEMV_TRAFFIC_RATIO,
            "algorithmic_bytes_per_launch": alg / n, "launch_us": sec / n * 1e6, "launches_timed": n * reps,
            "packed_stream_gbs": packed / sec / 1e9, "frac_of_8000": packed / sec / 1e9 / 8000.0}


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
    from rptc_b200.llama import LlamaConfig, RPTCLlama

    tp = args.workload.endswith("-tp")
    cfg = LlamaConfig(max_pos=args.prompt + max(3, args.warmup) + 2 * args.steps + 8, **cfg_kw)
    if tp:
        model = RPTCLlama(cfg, rows=1, seed=0, tp_world=world, tp_rank=rank, peer_allreduce=args.allreduce == "peer")
    else:
        model = RPTCLlama(cfg, rows=1, seed=rank)
    g = torch.Generator(device="cuda").manual_seed(42 + (0 if tp else rank))
    prompt = torch.randint(0, cfg.vocab, (args.prompt,), device="cuda", generator=g, dtype=torch.int32)
    model.reset()
    model.capture(pdl=True)
    for t in range(args.prompt):                           # the prompt goes through the decode step, token by token
        model.ids.copy_(prompt[t:t + 1])
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
    sampler = ClockSampler(local)
    barrier()
    pos_timed = model.pos.clone()          # both timed legs decode the same positions (same attention work)
    sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        model.step()
    b.record()
    b.synchronize()
    barrier()
    clocks = sampler.stop()
    ms = a.elapsed_time(b)
    # ---- end to end: host token in, host token out, every step ----
    # Single GPU / replicas: the mailbox loop of rptc_b200.llama.HostTokenLoop -- the host posts each step's token id
    # in pinned memory (8 bytes, read over PCIe by the step's first kernel) and polls the id the step's last kernel
    # writes back (8 bytes), keeping one graph launch queued ahead.  Tensor parallel: the step's first kernel reads a
    # pinned int32, the last writes a pinned int64, and the host synchronises the stream every step.
    first = int(model.ids.item())
    torch.cuda.synchronize()
    model.pos.copy_(pos_timed - 3)         # three untimed steps, then the positions of the device-resident leg
    model.sync_positions()
    if not tp:
        loop = model.host_loop()
        first = loop.run([first], 3)[-1][0]
        h2d, d2h = 8, 8
        barrier()
        t0 = time.perf_counter()
        loop.run([first], args.steps)
        torch.cuda.synchronize()
    else:
        host_in = torch.zeros(1, dtype=torch.int32).pin_memory()
        host_out = torch.zeros(1, dtype=torch.int64).pin_memory()
        host_in[0] = first
        model.bind_host_io(host_in, host_out)
        model.capture(pdl=True)
        h2d, d2h = 4, 8
        for _ in range(3):
            model.step()
            torch.cuda.current_stream().synchronize()
            host_in[0] = int(host_out[0])
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.step()
            torch.cuda.current_stream().synchronize()
            host_in[0] = int(host_out[0])
    e2e_s = time.perf_counter() - t0
    barrier()
    ops.device_status()

    t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        roof = gemv_roofline(model, torch)
        cpu_s, cores, sample = cpu_block_seconds(cfg_dims, 3)
        ctx = args.prompt + args.warmup + args.steps // 2
        bt = model.bytes_per_token(ctx)
        seqs = 1 if tp else world
        out = {"metric": METRIC if not tp else "2-bit Llama-2-70B-shape tensor-parallel decode tok/s (bs1)",
               "value": seqs * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if tp else "weak",
               "vs_baseline": None, "dtype": "f16", "data": "synthetic",
               "config": {"workload": args.workload, "code": "HASH S=8 K=2 L=16", "layout": "TILED", "incoherence": "RHT both sides",
                          "prompt": args.prompt, "batch_per_gpu": 1, "allreduce": (args.allreduce if tp else None), "parallelism": (f"tp{world}" if tp else ("replicas" if world > 1 else "single")),
                          "l2": "weights 1.6 GB per token exceed L2", "bytes_per_token": bt},
               "e2e": {"value": seqs * args.steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               "gpu_launches": model.launches_per_step * args.steps, "clocks": clocks, "roofline": roof,
               "cpu_baseline": {"value": 1.0 / cpu_s, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
               "token_stream_gbs": (bt["packed"] + bt["head"] + bt["kv"]) / (ms / args.steps * 1e-3) / 1e9}
        print(json.dumps(out))
    if world > 1:
        model.graph = None          # graphs that captured collectives must be gone before their communicator is torn down
        torch.cuda.synchronize()
        if getattr(model, "peer", None) is not None:
            model.peer.close()
        dist.barrier()
        dist.destroy_process_group()


WORKLOADS = {
    "llama2-7b-decode-bs1": (dict(), dict(hidden=4096, ffn=11008, layers=32, heads=32, kv_heads=32)),
    # the partitioned shape: tensor-parallel over all ranks (strong scaling), one all-reduce after o and down (--allreduce)
    "llama2-70b-tp": (dict(hidden=8192, layers=80, heads=64, kv_heads=8, ffn=28672),
                      dict(hidden=8192, ffn=28672, layers=80, heads=64, kv_heads=8)),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama2-7b-decode-bs1")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="tensor-parallel workloads: fused peer-memory all-reduce kernel, or NCCL")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt tokens pushed through the decode step before timing")
    args = ap.parse_args()
    cfg_kw, cfg_dims = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg_dims)
    else:
        run_ours(args, cfg_kw, cfg_dims)


if __name__ == "__main__":
    main()
