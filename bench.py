#!/usr/bin/env python
"""Benchmark of the B200-native quantized decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gemv|decode]

Prints ONE JSON line on rank 0.  For N > 1 it is launched by torch.distributed.run
(one rank per GPU).  See DESIGN.md, "Measurement", for what each field means.

Workload "gemv" (config 1 of BASELINE.json): the six q4_0 GEMV shapes, each as
one launch over a stack of distinct matrices totalling >= 512 MiB so that every
weight byte comes from HBM (inputs larger than the 126 MB L2; no flush needed).
A step is one pass over all six stacks.  value = algorithmic weight bytes / time.

`--impl reference` times the reference's own CPU path (its matvec, compiled from
the reference sources into oracle/_ref) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SWEEP = [(1536, 1536), (256, 1536), (8960, 1536), (1536, 8960), (151936, 1536), (11008, 2048)]   # (out, in)
STACK_BYTES = 512 << 20


def q4_bytes(rows, cols):
    return rows * cols * 18 // 32


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------ clocks sampling

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [l.split(",") for l in Path(self.f.name).read_text().splitlines() if l.count(",") >= 8]
        os.unlink(self.f.name)
        sm, reasons = [], set()
        for r in rows:
            try:
                sm.append(float(r[1])); out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------ reference arm (CPU)

def ref_matvec_sample(seconds_per_shape=2.0, shapes=None):
    """Time the reference's matvec (src/cpu_infer.cpp:22-32, all OpenMP threads) on one
    matrix per sweep shape.  Returns (GB/s over algorithmic q4_0 bytes, threads, description, ms per pass)."""
    sys.path.insert(0, str(ROOT / "tests"))
    import numpy as np
    import oracle_util as ou
    shapes = shapes or SWEEP
    kind = "reference" if ou.have_ref() else "port"
    rng = np.random.default_rng(0)
    tot_bytes, tot_s = 0, 0.0
    for rows, cols in shapes:
        nb = cols // 32
        raw = rng.integers(0, 256, size=(rows * nb, 18), dtype=np.uint8)
        raw[:, :2] = np.frombuffer(np.float16(rng.uniform(0.001, 0.01, rows * nb)).tobytes(), dtype=np.uint8).reshape(-1, 2)
        raw = raw.reshape(-1)
        x = rng.standard_normal(cols).astype(np.float32)
        y = np.empty(rows, np.float32)
        if kind == "reference":
            f = lambda: ou.ref().ref_matvec_q4_0(raw.ctypes.data, rows, cols, x.ctypes.data, y.ctypes.data)
        else:
            f = lambda: ou.lib().orc_matvec_f32(raw.ctypes.data, rows, cols, x.ctypes.data, y.ctypes.data)
        f()
        n, t0 = 0, time.perf_counter()
        while True:
            f(); n += 1
            dt = time.perf_counter() - t0
            if dt >= seconds_per_shape or n >= 2000:
                break
        tot_bytes += q4_bytes(rows, cols)
        tot_s += dt / n
    threads = ou.lib().orc_num_threads()
    return tot_bytes / tot_s / 1e9, threads, kind, tot_s * 1e3


def run_reference(args, rank):
    if rank != 0:
        return
    steps = max(1, args.steps)
    per_shape = min(2.0, 120.0 / (6 * (steps + args.warmup)))
    for _ in range(args.warmup):
        ref_matvec_sample(per_shape)
    vals, ms = [], []
    for _ in range(steps):
        v, threads, kind, m = ref_matvec_sample(per_shape)
        vals.append(v); ms.append(m)
    value = sum(vals) / len(vals)
    sample = "one matrix per sweep shape (1 of the GPU arm's stacked copies), fp32 activations, cpu_infer matvec"
    print(json.dumps({
        "impl": "reference", "metric": "q4_0 GEMV HBM GB/s (6-shape sweep, algorithmic q4_0 weight bytes / time)",
        "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(sum(ms) / len(ms), 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (reference CPU path dequantizes q4_0 rows to fp32)", "data": "synthetic",
        "config": {"workload": "gemv_sweep(config 1): " + ", ".join(f"{r}x{c}" for r, c in SWEEP)},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ our arm (GPU)

def build_stacks(ctx, torch, rank, world):
    """Per sweep shape: a stack of distinct random q4_0 matrices (>= STACK_BYTES on this rank),
    row-sharded across ranks by contiguous 32-row groups."""
    stacks = []
    g = torch.Generator(device="cuda"); g.manual_seed(1234 + rank)
    for rows, cols in SWEEP:
        groups = (rows + 31) // 32
        g0, g1 = groups * rank // world, groups * (rank + 1) // world
        my_rows = min(rows, g1 * 32) - g0 * 32
        nb = cols // 32
        count = max(1, -(-STACK_BYTES // q4_bytes(my_rows, cols)))
        n = count * my_rows * nb
        raw = torch.randint(0, 256, (n, 18), dtype=torch.uint8, device="cuda", generator=g)
        sc = (torch.rand(n, device="cuda", generator=g) * 0.009 + 0.001).to(torch.float16).view(torch.uint8).reshape(n, 2)
        raw[:, :2] = sc
        w = ctx.repack_q4_0_dev(raw.reshape(-1), my_rows, cols, count)
        del raw, sc
        x = torch.randn(cols, device="cuda", generator=g)
        xq = torch.empty(cols, dtype=torch.int8, device="cuda")
        xd = torch.empty(cols // 32, dtype=torch.float16, device="cuda")
        ctx.quant_q8(x, xq, xd)
        y = torch.empty((count, my_rows), dtype=torch.float32, device="cuda")
        stacks.append(dict(w=w, xq=xq, xd=xd, y=y, x_host=x.cpu().numpy(), rows=my_rows, cols=cols, count=count,
                           bytes=q4_bytes(my_rows, cols) * count))
    torch.cuda.synchronize()
    return stacks


def run_ours(args, rank, world, local_rank):
    import numpy as np
    import torch
    import __graft_entry__ as ge
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = ge.load_package()
    ctx = pkg.Context(local_rank)
    ctx.use_torch_stream()
    stacks = build_stacks(ctx, torch, rank, world)
    step_bytes = sum(s["bytes"] for s in stacks)

    def step():
        for s in stacks:
            ctx.gemv_q4_q8(s["w"], s["xq"], s["xd"], s["y"])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # --- timed region: K steps, CUDA events on the launching stream
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stacks) + 1)] for _ in range(args.steps)]
    barrier()
    t_wall0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(args.steps):
        ev[k][0].record()
        for i, s in enumerate(stacks):
            ctx.gemv_q4_q8(s["w"], s["xq"], s["xd"], s["y"])
            ev[k][i + 1].record()
    e1.record()
    barrier()
    ctx.sync()
    wall_ms = (time.perf_counter() - t_wall0) * 1e3
    total_ms = e0.elapsed_time(e1)
    # per-kernel durations (one launch per stack) for the roofline of the dominant kernel
    kern_ms = [sum(ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(args.steps)) / args.steps for i in range(len(stacks))]
    # --- end to end through the host-buffer entry point: H2D of x, D2H of y inside the timed region
    e2e_steps = max(1, min(args.steps, 5))
    youts = [np.empty((s["count"], s["rows"]), np.float32) for s in stacks]
    for s, yo in zip(stacks, youts):
        ctx.gemv_q4_f32_host(s["w"], s["x_host"], yo)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for s, yo in zip(stacks, youts):
            ctx.gemv_q4_f32_host(s["w"], s["x_host"], yo)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    clocks = sampler.stop() if sampler else None

    if dist is not None:
        t = torch.tensor([total_ms, e2e_ms, float(step_bytes)], device="cuda", dtype=torch.float64)
        tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, all_bytes = float(tmax[0]), float(tmax[1]), float(tsum[2])
    else:
        all_bytes = float(step_bytes)
    if rank != 0:
        return
    ms_per_step = total_ms / args.steps
    value = all_bytes / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()
    # dominant kernel: the GEMV (the only kernel of this workload); achieved over all six launches of a step
    ach = step_bytes / (sum(kern_ms) * 1e-3) / 1e9
    cpu_v, cpu_threads, cpu_kind, _ = ref_matvec_sample(1.5)
    out = {
        "metric": "q4_0 GEMV HBM GB/s (6-shape sweep, algorithmic q4_0 weight bytes / time)",
        "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int4 dot products (dp4a, int32) with fp16 block scales, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "gemv_sweep(config 1): " + ", ".join(f"{r}x{c}" for r, c in SWEEP),
                   "stack_bytes_per_shape_per_gpu": STACK_BYTES, "l2": "inputs larger than L2 (each launch streams >= 512 MiB of distinct weights)",
                   "sharding": "rows of every matrix split across ranks by 32-row groups, no collective"},
        "roofline": {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4),
                     "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})", "traffic": None,
                     "kernel": "gemv_q4_q8_kernel", "per_shape_gbs": {f"{r}x{c}": round(s["bytes"] / (m * 1e-3) / 1e9, 1)
                                                                      for (r, c), s, m in zip(SWEEP, stacks, kern_ms)}},
        "cpu_baseline": {"value": round(cpu_v, 3), "unit": "GB/s", "cores": cpu_threads, "kind": cpu_kind,
                         "sample": "one matrix per sweep shape, ~1.5 s each, reference matvec (fp32 activations) on all host threads"},
        "e2e": {"value": round(all_bytes / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": int(sum(s["cols"] * 4 for s in stacks)),
                "d2h_bytes_per_step": int(sum(s["count"] * s["rows"] * 4 for s in stacks)),
                "api": "mi_gemv_q4_f32_host (host x in, host y out; weights resident)"},
        "gpu_launches": args.steps * len(stacks),
        "clocks": clocks,
        "wall_ms_timed_region": round(wall_ms, 2),
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--stack-mb", type=int, default=512, help="distinct weight bytes per shape per GPU (MiB); small values are for profiler captures")
    ap.add_argument("--shapes", default="", help="comma list like 8960x1536 to restrict the sweep (profiler captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    global STACK_BYTES, SWEEP
    STACK_BYTES = args.stack_mb << 20
    if args.shapes:
        SWEEP = [tuple(int(v) for v in t.split("x")) for t in args.shapes.split(",")]
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
