"""Benchmark of the recurrent-scan hot path: time-varying diagonal scan, forward + adjoint.

Workload ("C2"): B=64, T=4096, D=256 float32 per GPU, a_t = sigmoid(N(2,1)), b_t ~ N(0,1),
h0 = 0, upstream gradient ~ N(0,1), all synthetic and seeded.  One step = one forward scan
(a, b -> h) plus one adjoint scan (g, a, h -> ga, gb): 8 tensor passes of 268.4 MB, i.e. 2147.5 MB
of compulsory HBM traffic, the figure every GB/s number below is computed from.  With N GPUs every
rank scans its own 64 sequences (weak scaling; the scan has no collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line: `value` is device-resident throughput (inputs already in HBM), `e2e` the
same metric through the public API from pinned HOST buffers with the host<->device copies inside
the timed region, `roofline` the dominant kernel (the adjoint) against the measured HBM peak, and
`cpu_baseline` the CPU oracle (a C port of the reference's CPU kernels) on the host cores.
`--impl reference` times that CPU port alone and prints the same line shape.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, T, D = 64, 4096, 256
TENSOR_BYTES = B * T * D * 4
FWD_BYTES = 3 * TENSOR_BYTES  # a, b -> h
BWD_BYTES = 5 * TENSOR_BYTES  # g, a, h -> ga, gb
STEP_BYTES = FWD_BYTES + BWD_BYTES
ADJOINT_DRAM_TRAFFIC_BYTES = 805_204_224 + 495_119_360
METRIC = "scan GB/s (fwd+bwd)"
WORKLOAD = "C2: time-varying diagonal scan fwd+bwd, B=64 T=4096 D=256 fp32 per GPU, h0=0"


def _peaks():
    """Measured HBM peak of this pool's B200s, else the stated fallback."""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clock/throttle samples every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
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
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample(seconds_target: float = 12.0, steps: int = 1, warmup: int = 1):
    """Time the CPU oracle (float32, all host threads) on a slice of the workload.

    The slice is `rows` of the 64 sequences, grown until one fwd+bwd pass takes a measurable time;
    throughput in GB/s is per algorithmic byte, so it compares directly with the GPU figure.
    """
    import numpy as np
    from oracle import oracle as O

    O.build()
    rng = np.random.default_rng(0)
    rows = 8
    a = (1.0 / (1.0 + np.exp(-(rng.standard_normal((rows, T, D), dtype=np.float32) + 2.0)))).astype(np.float32)
    b = rng.standard_normal((rows, T, D), dtype=np.float32)
    g = rng.standard_normal((rows, T, D), dtype=np.float32)

    def one():
        h = O.sel_fwd(a, b, None)
        O.sel_bwd(g, a, h, None)

    for _ in range(max(1, warmup)):
        one()
    times = []
    t_end = time.perf_counter() + seconds_target
    while len(times) < steps or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
        if len(times) >= steps and time.perf_counter() >= t_end:
            break
    sec = statistics.median(times)
    gbs = STEP_BYTES * rows / B / sec / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{rows} of {B} sequences (T={T}, D={D}), fwd+bwd, median of {len(times)} passes of "
                      f"{sec * 1e3:.1f} ms; C port of the reference's selective_c kernels, OpenMP"}, sec, rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec, rows = cpu_sample(seconds_target=10.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3 * B / rows, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU port of the reference kernels on the host cores; "
                   "ms_per_step is the sample time scaled to the full 64 sequences"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    import tsfast_b200
    from tsfast_b200.scan_backends import selective_b200 as sel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the product has no CPU path; use --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    a = torch.sigmoid(torch.randn(B, T, D, device=dev, generator=gen) + 2.0)
    b = torch.randn(B, T, D, device=dev, generator=gen)
    g = torch.randn(B, T, D, device=dev, generator=gen)

    def step():
        h = sel.forward(a, b, None)
        return sel.backward(g, a, h, None)

    for _ in range(args.warmup):
        step()
    barrier()

    # ---- device-resident throughput: K steps between two events, max over ranks
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clock_rec = clocks.stop() if rank == 0 else None

    # ---- per-kernel durations: n back-to-back launches of one kernel between two events
    n = max(3, min(args.steps, 10))
    h = sel.forward(a, b, None)
    s0, s1, s2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    torch.cuda.synchronize()
    s0.record()
    for _ in range(n):
        h = sel.forward(a, b, None)
    s1.record()
    for _ in range(n):
        sel.backward(g, a, h, None)
    s2.record()
    torch.cuda.synchronize()
    fwd_ms, bwd_ms = s0.elapsed_time(s1) / n, s1.elapsed_time(s2) / n

    e2e_ms = float("nan")
    if not args.kernel_only:
        e2e_ms = _e2e(args, torch, tsfast_b200, dev, a, b, g, barrier)

    times = torch.tensor([ms, e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(x) for x in times.tolist())
    _report(args, world, rank, ms, e2e_ms, fwd_ms, bwd_ms, clock_rec)
    if world > 1:
        dist.destroy_process_group()


def _e2e(args, torch, tsfast_b200, dev, a, b, g, barrier):
    """Same step through the public API from pinned host buffers, copies inside the timed region."""
    ha, hb, hg = (torch.empty(B, T, D, pin_memory=True).copy_(t) for t in (a, b, g))
    ho, hga, hgb = (torch.empty(B, T, D, pin_memory=True) for _ in range(3))

    def e2e_step():
        da = ha.to(dev, non_blocking=True).requires_grad_()
        db = hb.to(dev, non_blocking=True).requires_grad_()
        dg = hg.to(dev, non_blocking=True)
        out = tsfast_b200.selective_recurrence(da, db)
        out.backward(dg)
        ho.copy_(out.detach(), non_blocking=True)
        hga.copy_(da.grad, non_blocking=True)
        hgb.copy_(db.grad, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t1.record()
    barrier()
    return t0.elapsed_time(t1) / e2e_steps


def _report(args, world, rank, ms, e2e_ms, fwd_ms, bwd_ms, clock_rec):
    if rank == 0:
        peak, peak_src = _peaks()
        value = STEP_BYTES * world / (ms * 1e-3) / 1e9
        bwd_gbs = BWD_BYTES / (bwd_ms * 1e-3) / 1e9
        fwd_gbs = FWD_BYTES / (fwd_ms * 1e-3) / 1e9
        base = None
        if world == 1 and not args.no_cpu and not args.kernel_only:
            base = cpu_sample()[0]
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "algorithmic_bytes_per_step_per_gpu": STEP_BYTES,
                       "state_elements_per_s": round(2 * B * T * D * world / (ms * 1e-3)),
                       "l2": "each of the 8 streamed tensors is 268 MB, larger than the 126 MB L2; no flush needed",
                       "sharding": "independent sequences per rank, no collective"},
            "roofline": {"bound": "hbm", "kernel": "diag_stream_kernel<float, varying, adjoint> (b200_sel_bwd)",
                         "achieved": round(bwd_gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(bwd_gbs / peak, 4), "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": BWD_BYTES, "ms_per_launch": round(bwd_ms, 4),
                         "forward_kernel": {"achieved": round(fwd_gbs, 1), "frac": round(fwd_gbs / peak, 4),
                                            "algorithmic_bytes_per_launch": FWD_BYTES,
                                            "ms_per_launch": round(fwd_ms, 4)}},
            "cpu_baseline": base,
            "e2e": None if args.kernel_only else {
                "value": round(STEP_BYTES * world / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": 3 * TENSOR_BYTES, "d2h_bytes_per_step": 3 * TENSOR_BYTES,
                "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": 2 * args.steps,
            "clocks": clock_rec,
        }
        # dram__bytes_read.sum + dram__bytes_write.sum of one adjoint launch at this workload, from the
        # ncu capture summarised in profiles/sel_scan_c2_ncu_full.md
        line["roofline"]["traffic"] = ADJOINT_DRAM_TRAFFIC_BYTES
        print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (no end-to-end or CPU leg): the command profiled under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
