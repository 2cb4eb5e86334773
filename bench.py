"""Benchmark of the recurrent-scan hot path: time-varying diagonal scan, forward + adjoint.

Workload ("C2"): B=64, T=4096, D=256 float32 per GPU, a_t = sigmoid(N(2,1)), b_t ~ N(0,1),
h0 = 0, upstream gradient ~ N(0,1), all synthetic and seeded.  One step = one forward scan
(a, b -> h) plus one adjoint scan (g, a, h -> ga, gb): 8 tensor passes of 268.4 MB, i.e. 2147.5 MB
of compulsory HBM traffic, the figure every GB/s number below is computed from.  With N GPUs every
rank scans its own 64 sequences (weak scaling; the scan has no collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload C1..C5|G|V|P]

Prints ONE JSON line: `value` is device-resident throughput (inputs already in HBM), `e2e` the
same metric through the public API from pinned HOST buffers with the host<->device copies inside
the timed region, `roofline` the dominant kernel (the adjoint) against the measured HBM peak, and
`cpu_baseline` the reference's own CPU kernel (tsfast's generated-C++ `selective_c` backend, run
from the unmodified copy under oracle/_ref) on the host cores; where that copy is missing or does
not build, the C port of the same kernel (oracle/) is timed instead and the line says so.
`--impl reference` times that CPU path alone and prints the same line shape.
The default run also measures, kernel-only and with the same event method, the other scans
(`config.workloads`: C1 complex LRU scan, C3 Mamba section, C4 all-pole filter), the DeepLRU
data-parallel training step (`config.c5`) and, on one GPU, the reference's own Triton kernels on
the same device (`config.triton`, `config.vs_triton`).
`--workload C1|C3|C4|C5|G|V|P` prints a full line for one of the other configurations (G the fused
dynoNet block, V the Mamba causal conv + SiLU, P the tensor-core projection GEMM); C2 is the headline.

A rank that fails prints one `{"rank", "error", "where"}` JSON line to stdout and stderr before it
exits non-zero.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, T, D = 64, 4096, 256
C2_SHAPE = (B, T, D)
TENSOR_BYTES = B * T * D * 4
FWD_BYTES = 3 * TENSOR_BYTES  # a, b -> h
BWD_BYTES = 5 * TENSOR_BYTES  # g, a, h -> ga, gb
STEP_BYTES = FWD_BYTES + BWD_BYTES
E2E_CHUNKS = 8  # batch slices the end-to-end step is pipelined over
E2E_STREAMS = 3  # streams the slices are issued on, round-robin (one pinned slot per stream and direction)
ADJOINT_DRAM_TRAFFIC_BYTES = 805_204_224 + 495_119_360  # ncu dram__bytes read + write of one adjoint launch
METRIC = "scan GB/s (fwd+bwd)"
WORKLOAD = "C2: time-varying diagonal scan fwd+bwd, B=64 T=4096 D=256 fp32 per GPU, h0=0"


def _emit(line: dict) -> None:
    """Print the result as the LAST line of stdout: libraries that write through C stdio (NCCL's
    version banner) are flushed first, so nothing buffered can land after the JSON line."""
    import ctypes

    sys.stdout.flush()
    try:
        ctypes.CDLL(None).fflush(None)
    except OSError:
        pass
    print(json.dumps(line), flush=True)


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


def _time_cpu(fn, steps, warmup, seconds_target):
    """Median wall time of fn() over at least `steps` passes, stopping after about seconds_target."""
    for _ in range(max(1, warmup)):
        fn()
    times, t_end = [], time.perf_counter() + seconds_target
    while len(times) < max(1, steps) or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


# ----------------------------------------------------------------------------- CPU arm
def _host_threads() -> int:
    return len(os.sched_getaffinity(0))  # torchrun exports OMP_NUM_THREADS=1; use every core we may


def _import_reference():
    """tsfast from the unmodified copy under oracle/_ref: the baseline legs time its kernels, and the
    full-model workload (C5) uses its DeepLRU as the caller of this package's scans.  The package
    tsfast_b200 itself never imports it."""
    ref = ROOT / "oracle" / "_ref"
    if not (ref / "tsfast" / "models" / "_core" / "scan.py").exists():
        raise ImportError("oracle/_ref holds no tsfast copy (python oracle/make_ref.py <checkout>)")
    # tsfast compiles its C++ kernels at run time with $CXX; the system compiler is named because
    # some images export one that cannot link OpenMP
    for var, exe in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):
        if os.path.exists(exe):
            os.environ[var] = exe
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    import tsfast.models  # noqa: F401
    import tsfast.models._core.scan as ref_scan
    from tsfast.models import use_backend

    return ref_scan, use_backend


def _cpu_reference(steps: int, warmup: int, seconds_target: float):
    """The reference's own CPU path for C2: `selective_recurrence` under `use_backend("c")` (tsfast's
    generated-C++ kernel, `_core/scan_backends/selective_c.py`) on all 64 sequences, forward +
    backward on fresh leaves every pass, all host threads."""
    import torch

    ref_scan, use_backend = _import_reference()
    torch.set_num_threads(_host_threads())
    gen = torch.Generator().manual_seed(0)
    a0 = torch.sigmoid(torch.randn(B, T, D, generator=gen) + 2.0)
    b0 = torch.randn(B, T, D, generator=gen)
    g = torch.randn(B, T, D, generator=gen)

    def one():
        a, b = a0.clone().requires_grad_(), b0.clone().requires_grad_()
        with use_backend("c"):
            ref_scan.selective_recurrence(a, b).backward(g)

    with use_backend("c"):  # the first call compiles the kernel; a backend that cannot build warns and falls back
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("error", RuntimeWarning)
            ref_scan.selective_recurrence(a0[:1, :8], b0[:1, :8])
    sec, cnt = _time_cpu(one, steps, warmup, seconds_target)
    return {"value": round(STEP_BYTES / sec / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "reference",
            "sample": f"all {B} sequences (T={T}, D={D}), fwd+bwd on fresh leaves, median of {cnt} passes of {sec * 1e3:.1f} ms; "
                      "tsfast's own generated-C++ selective_c backend through selective_recurrence under use_backend('c')"}, sec


def _cpu_port(steps: int, warmup: int, seconds_target: float, why: str):
    """Fallback: the C port of the same kernel (oracle/), on 8 of the 64 sequences, scaled."""
    import numpy as np
    from oracle import oracle as O

    O.build()
    O.set_num_threads(_host_threads())
    rng = np.random.default_rng(0)
    rows = 8
    a = (1.0 / (1.0 + np.exp(-(rng.standard_normal((rows, T, D), dtype=np.float32) + 2.0)))).astype(np.float32)
    b = rng.standard_normal((rows, T, D), dtype=np.float32)
    g = rng.standard_normal((rows, T, D), dtype=np.float32)

    def one():
        h = O.sel_fwd(a, b, None)
        O.sel_bwd(g, a, h, None)

    sec, cnt = _time_cpu(one, steps, warmup, seconds_target)
    sec = sec * B / rows
    return {"value": round(STEP_BYTES / sec / 1e9, 3), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{rows} of {B} sequences (T={T}, D={D}) scaled to {B}, fwd+bwd, median of {cnt} passes; C port of the "
                      f"reference's selective_c kernel, OpenMP (the reference's own backend was not usable: {why})"}, sec


def cpu_sample(seconds_target: float = 12.0, steps: int = 3, warmup: int = 2):
    """CPU baseline of the C2 step on the host cores: the reference's own kernel, else the port."""
    try:
        return _cpu_reference(steps, warmup, seconds_target)
    except Exception as e:  # no copy of the reference here, or its C++ backend does not build on this host
        return _cpu_port(steps, warmup, seconds_target, f"{type(e).__name__}: {str(e)[:120]}")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec = cpu_sample(seconds_target=20.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "the reference's CPU implementation of the path on the host cores"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


# ----------------------------------------------------------------------------- GPU arm
def _dist_setup():
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the product has no CPU path; use --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    return torch, dist, world, rank, local, dev, barrier


def _make_timed(torch, dev):
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, n):
        """Mean device time of fn() over n calls.  A 256 MB buffer is rewritten four times before
        every call: that flushes L2 and keeps the GPU busy while the host enqueues fn(), so the
        two events bracket the call's device work and not the host's launch path."""
        tot = 0.0
        for _ in range(n):
            for _ in range(4):
                flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / n

    return timed


def run_gpu(args):
    torch, dist, world, rank, local, dev, barrier = _dist_setup()

    import tsfast_b200
    from tsfast_b200.scan_backends import selective_b200 as sel

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

    e2e_ms, e2e_info = float("nan"), {}
    if not args.kernel_only:
        e2e_ms, e2e_info = _e2e(args, torch, tsfast_b200, dev, a, b, g, barrier)
    del a, b, g, h
    torch.cuda.empty_cache()

    others, c5, triton = {}, None, None
    if not args.kernel_only:
        timed = _make_timed(torch, dev)
        for name in ("C1", "C3", "C4"):
            others[name] = _kernel_only(name, torch, dev, rank, timed, max(10, min(args.steps, 20)),
                                        with_cpu=world == 1 and rank == 0 and not args.no_cpu)
            torch.cuda.empty_cache()
        try:
            c5 = _c5_measure(torch, dist, dev, world, rank, local, barrier, steps=max(5, min(args.steps, 10)), warmup=3)
            if world == 1:  # the same step with the GEMMs left to PyTorch: what the tensor-core projections buy
                c5["ms_per_step_gemms_in_pytorch"] = _c5_measure(torch, dist, dev, world, rank, local, barrier, steps=5,
                                                                 warmup=3, plain_gemms=True)["ms_per_step"]
        except ImportError as e:  # no tsfast copy on this machine: the step's caller is missing, not the kernels
            c5 = None
            others["C5"] = {"unavailable": f"{e}"[:200]}
        torch.cuda.empty_cache()
        if world == 1 and not args.no_triton:
            triton = _triton_baseline(torch, dev, timed)
            torch.cuda.empty_cache()
    sys.stdout.flush()

    times = torch.tensor([ms, e2e_ms] + ([c5["ms_per_step"]] if c5 else []), device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    vals = [float(x) for x in times.tolist()]
    ms, e2e_ms = vals[0], vals[1]
    if c5:
        c5["ms_per_step"] = round(vals[2], 3)
        c5["windows_per_s"] = round(c5["windows_per_gpu"] * world / (vals[2] * 1e-3), 1)
    _report(args, world, rank, ms, e2e_ms, e2e_info, fwd_ms, bwd_ms, clock_rec, others, c5, triton)
    if world > 1:
        dist.destroy_process_group()


def _e2e(args, torch, tsfast_b200, dev, a, b, g, barrier):
    """Same step through the public API from pinned host buffers, copies inside the timed region.

    The sequences of a batch are independent, so the step is issued as E2E_CHUNKS batch slices
    round-robin on E2E_STREAMS streams: the host-to-device copy of one slice, the scans of another and
    the device-to-host copy of a third overlap, which keeps both PCIe directions busy.  Every slice
    copies its full a, b, g in and its full h, ga, gb out, so every byte of the batch crosses PCIe in
    both directions each step.  Host memory is a ring: each stream owns one pinned input slot (a, b, g
    of one slice) and one pinned output slot, reused by every slice issued on that stream (stream order
    keeps the reuse safe).  Slot s holds the rows of slice s, so slice k computes on the data of slice
    k mod E2E_STREAMS; its result is checked against the device-resident call on the same rows.
    """
    rows = B // E2E_CHUNKS
    pin = lambda: torch.empty(rows, T, D, pin_memory=True)  # noqa: E731
    slots_in = [[pin().copy_(t[s * rows:(s + 1) * rows]) for t in (a, b, g)] for s in range(E2E_STREAMS)]
    slots_out = [[pin() for _ in range(3)] for _ in range(E2E_STREAMS)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(E2E_STREAMS)]

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        for s_ in streams:
            s_.wait_stream(cur)
        for k in range(E2E_CHUNKS):
            s = k % E2E_STREAMS
            ha, hb, hg = slots_in[s]
            ho, hga, hgb = slots_out[s]
            with torch.cuda.stream(streams[s]):
                da = ha.to(dev, non_blocking=True).requires_grad_()
                db = hb.to(dev, non_blocking=True).requires_grad_()
                dg = hg.to(dev, non_blocking=True)
                out = tsfast_b200.selective_recurrence(da, db)
                out.backward(dg)
                ho.copy_(out.detach(), non_blocking=True)
                hga.copy_(da.grad, non_blocking=True)
                hgb.copy_(db.grad, non_blocking=True)
        for s_ in streams:
            cur.wait_stream(s_)

    def copy_only_step():  # the same bytes over PCIe with no kernels: the ceiling of this host path
        cur = torch.cuda.current_stream(dev)
        for s_ in streams:
            s_.wait_stream(cur)
        for k in range(E2E_CHUNKS):
            s = k % E2E_STREAMS
            with torch.cuda.stream(streams[s]):
                dd = [h_.to(dev, non_blocking=True) for h_ in slots_in[s]]
                for h_, d_ in zip(slots_out[s], dd):
                    h_.copy_(d_, non_blocking=True)
        for s_ in streams:
            cur.wait_stream(s_)

    def clock(fn, n):
        fn()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        barrier()
        return t0.elapsed_time(t1) / n

    e2e_steps = max(2, min(args.steps, 5))
    ms = clock(e2e_step, e2e_steps)
    # the pipelined path must deliver the numbers of the device-resident call on the same rows
    worst, same_bits = 0.0, True
    for s in range(E2E_STREAMS):
        sl = slice(s * rows, (s + 1) * rows)
        da, db = a[sl].clone().requires_grad_(), b[sl].clone().requires_grad_()
        ref = tsfast_b200.selective_recurrence(da, db)
        ref.backward(g[sl])
        for got, want in zip(slots_out[s], (ref.detach(), da.grad, db.grad)):
            got = got.to(dev)
            err = ((got - want).abs().max() / want.abs().max()).item()
            worst = max(worst, err)
            same_bits = same_bits and bool(torch.equal(got, want))
    if not worst < 1e-4:
        raise RuntimeError(f"end-to-end result differs from the device-resident result: max|a-b|/max|b| = {worst:.3e}")
    copy_ms = clock(copy_only_step, e2e_steps)
    return ms, {"check_max_rel_err": worst, "check_bitwise_equal": same_bits, "copy_only_ms_per_step": round(copy_ms, 3),
                "pinned_host_bytes": 6 * E2E_STREAMS * rows * T * D * 4}


def _reference_cpu_leg(wl, torch, seconds_target: float = 3.0):
    """The reference's own CPU implementation of a workload (its `ref_cpu` closure) on a few batch
    rows, scaled to the whole batch; None with the reason when that path cannot run here."""
    try:
        rows = wl.get("ref_rows", wl["sample_rows"])
        torch.set_num_threads(_host_threads())
        one, what = wl["ref_cpu"](rows)
        one()  # compiles the reference's C/C++ kernel on first use
        sec, cnt = _time_cpu(one, 1, 1, seconds_target)
        step_bytes = wl["fwd_bytes"] + wl["bwd_bytes"]
        return {"value": round(step_bytes * rows / wl["rows"] / sec / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(),
                "kind": "reference", "sample": f"{rows} of {wl['rows']} batch rows, fwd+bwd on fresh leaves, median of {cnt} "
                                               f"passes of {sec * 1e3:.1f} ms; {what}"}, None
    except Exception as e:
        return None, f"the reference's own path was not usable: {type(e).__name__}: {str(e)[:120]}"


def _kernel_only(name, torch, dev, rank, timed, steps, with_cpu=False):
    """Forward and adjoint kernels of one of the other configurations, device-resident, event-timed
    (with_cpu: the reference's CPU path for the same workload timed beside them)."""
    wl = _workload(name, torch, dev, rank, host_buffers=False)
    keep = {}

    def step():
        keep["o"] = wl["fwd"]()
        wl["bwd"](keep["o"])

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    ms = timed(step, steps)
    fwd_ms = timed(lambda: keep.__setitem__("o", wl["fwd"]()), steps)
    bwd_ms = timed(lambda: wl["bwd"](keep["o"]), steps)
    peak, _ = _peaks()
    step_bytes = wl["fwd_bytes"] + wl["bwd_bytes"]
    rec = {"workload": wl["desc"], "gbs": round(step_bytes / ms / 1e6, 1), "ms_per_step": round(ms, 4), "steps": steps,
           "fwd_ms": round(fwd_ms, 4), "bwd_ms": round(bwd_ms, 4),
           "fwd_frac": round(wl["fwd_bytes"] / fwd_ms / 1e6 / peak, 4), "bwd_frac": round(wl["bwd_bytes"] / bwd_ms / 1e6 / peak, 4),
           "algorithmic_bytes_per_step": step_bytes, "traffic": wl.get("traffic"),
           "state_elements_per_s": round(wl["elems"] / (ms * 1e-3))}
    if with_cpu and "ref_cpu" in wl:
        base, why = _reference_cpu_leg(wl, torch)
        rec["cpu_baseline"] = base if base is not None else {"unavailable": why}
    return rec


def _triton_baseline(torch, dev, timed):
    """The reference's own GPU kernels (tsfast's Triton backends, unmodified copy under oracle/_ref) on
    this device, same inputs, same event method: the kernels this library replaces."""
    try:
        _import_reference()
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    out = {}
    for name in ("C1", "C2", "C3", "C4"):
        try:
            wl = _workload(name, torch, dev, 0, host_buffers=False, impl="triton")
            keep = {}

            def step():
                keep["o"] = wl["fwd"]()
                wl["bwd"](keep["o"])

            for _ in range(3):  # the first calls compile and autotune
                step()
            torch.cuda.synchronize()
            ms = timed(step, 10)
            out[name] = {"ms_per_step": round(ms, 4), "gbs": round((wl["fwd_bytes"] + wl["bwd_bytes"]) / ms / 1e6, 1)}
        except Exception as e:  # Triton could not compile or run this kernel on this device
            out[name] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        torch.cuda.empty_cache()
    return out


def _report(args, world, rank, ms, e2e_ms, e2e_info, fwd_ms, bwd_ms, clock_rec, others, c5, triton):
    if rank != 0:
        return
    peak, peak_src = _peaks()
    value = STEP_BYTES * world / (ms * 1e-3) / 1e9
    bwd_gbs = BWD_BYTES / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = FWD_BYTES / (fwd_ms * 1e-3) / 1e9
    base = None
    if world == 1 and not args.no_cpu and not args.kernel_only:
        base = cpu_sample()[0]
    config = {"workload": WORKLOAD, "algorithmic_bytes_per_step_per_gpu": STEP_BYTES,
              "state_elements_per_s": round(2 * B * T * D * world / (ms * 1e-3)),
              "l2": "each of the 8 streamed tensors is 268 MB, larger than the 126 MB L2; no flush needed",
              "sharding": "independent sequences per rank, no collective"}
    if others:
        config["workloads"] = others
    if c5:
        config["c5"] = c5
    if triton is not None:
        config["triton"] = triton
        ours = dict({k: v["gbs"] for k, v in others.items() if "gbs" in v}, C2=value)
        config["vs_triton"] = {k: round(ours[k] / v["gbs"], 2) for k, v in triton.items()
                               if isinstance(v, dict) and "gbs" in v and k in ours}
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "roofline": {"bound": "hbm", "kernel": "diag_stream_kernel<float, varying, adjoint> (b200_sel_bwd)",
                     "achieved": round(bwd_gbs, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(bwd_gbs / peak, 4), "traffic": ADJOINT_DRAM_TRAFFIC_BYTES, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": BWD_BYTES, "ms_per_launch": round(bwd_ms, 4),
                     "forward_kernel": {"achieved": round(fwd_gbs, 1), "frac": round(fwd_gbs / peak, 4),
                                        "algorithmic_bytes_per_launch": FWD_BYTES,
                                        "ms_per_launch": round(fwd_ms, 4)}},
        "cpu_baseline": base,
        "e2e": None if args.kernel_only else dict({
            "value": round(STEP_BYTES * world / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
            "h2d_bytes_per_step": 3 * TENSOR_BYTES, "d2h_bytes_per_step": 3 * TENSOR_BYTES,
            "ms_per_step": round(e2e_ms, 3),
            "how": f"{E2E_CHUNKS} batch slices round-robin on {E2E_STREAMS} streams (copies overlap the scans and each "
                   "other); one pinned slot per stream and direction"}, **e2e_info),
        "gpu_launches": 2 * args.steps,  # device-resident region; the end-to-end region launches 2 per slice
        "clocks": clock_rec,
    }
    _emit(line)


# ----------------------------------------------------------------------------- other workloads
# C1, C3, C4 (one scan each) and C5 (DeepLRU training step).  Same JSON line as the default
# workload; per-step events, with an L2 flush between steps where the working set fits in L2.
def _workload(name, torch, dev, rank, host_buffers=True, impl="b200"):
    """Returns dict(desc, fwd_bytes, bwd_bytes, elems, fwd(), bwd(out), e2e(), cpu(rows)->sec, rows, flush).

    `host_buffers=False` skips the pinned host copies the end-to-end leg needs.  `impl="triton"`
    binds fwd/bwd to the reference's Triton modules (same op names and arguments) instead of this
    package's: the baseline leg."""
    import numpy as np

    import tsfast_b200

    if impl == "triton":
        from tsfast.models._core.scan_backends import diagonal_triton as diagonal_b200
        from tsfast.models._core.scan_backends import selective_triton as selective_b200
        from tsfast.models.architectures.dynonet import allpole_triton as allpole_b200
        from tsfast.models.architectures.mamba import mamba_triton as mamba_b200
    else:
        from tsfast_b200 import allpole_b200, mamba_b200
        from tsfast_b200.scan_backends import diagonal_b200, selective_b200

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)  # noqa: E731

    def pin(t):
        if not host_buffers:
            return None
        return torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)

    if name == "C2":
        a = torch.sigmoid(rn(*C2_SHAPE) + 2.0)
        b, g = rn(*C2_SHAPE), rn(*C2_SHAPE)
        return dict(desc=WORKLOAD, fwd_bytes=FWD_BYTES, bwd_bytes=BWD_BYTES, elems=2 * TENSOR_BYTES // 4, rows=C2_SHAPE[0], flush=False,
                    dtype="f32", launches=2, fwd=lambda: selective_b200.forward(a, b, None),
                    bwd=lambda o: selective_b200.backward(g, a, o, None))
    if name == "C1":
        M, L, N = 16, 1000, 64
        r = torch.rand(N, device=dev, generator=gen) * 0.099 + 0.9
        th = torch.rand(N, device=dev, generator=gen) * (np.pi / 10)
        lam1 = torch.polar(r, th)
        lam = lam1.expand(M, N).contiguous()
        cn = lambda *s: torch.complex(rn(*s), rn(*s)) * (0.5**0.5)  # noqa: E731
        v, g, x0 = cn(M, L, N), cn(M, L, N), cn(M, N) * (0.1**0.5)
        E = M * L * N * 8
        hv, hg, hx0 = pin(v), pin(g), pin(x0)
        ho, hgv = pin(v), pin(v)

        def e2e():
            dv, dx0 = hv.to(dev, non_blocking=True).requires_grad_(), hx0.to(dev, non_blocking=True).requires_grad_()
            l1 = lam1.clone().requires_grad_()
            out = tsfast_b200.diagonal_recurrence(l1, dv, dx0)
            out.backward(hg.to(dev, non_blocking=True))
            ho.copy_(out.detach(), non_blocking=True)
            hgv.copy_(dv.grad, non_blocking=True)
            return l1.grad.cpu()

        def cpu(rows):
            from oracle import oracle as O
            a_, v_, g_, x_ = (t[:rows].cpu().numpy() for t in (lam, v, g, x0))
            return lambda: O.diag_bwd(g_, a_, O.diag_fwd(a_, v_, x_), x_)

        def ref_cpu(rows):  # tsfast's generated-C++ diagonal kernel (scan_backends/diagonal_c.py) through its public function
            ref_scan, use_backend = _import_reference()
            l_, v_, g_, x_ = lam1.cpu(), v[:rows].cpu(), g[:rows].cpu(), x0[:rows].cpu()

            def one():
                lq, vq, xq = l_.clone().requires_grad_(), v_.clone().requires_grad_(), x_.clone().requires_grad_()
                with use_backend("c"):
                    ref_scan.diagonal_recurrence(lq, vq, xq).backward(g_)
            return one, "diagonal_recurrence under use_backend('c') (tsfast's generated-C++ diagonal_c kernel)"

        return dict(desc="C1: complex LRU diagonal scan fwd+bwd, B=16 T=1000 D=64 complex64, carry-in x0", ref_cpu=ref_cpu,
                    fwd_bytes=2 * E, bwd_bytes=3 * E, elems=2 * M * L * N, rows=M, sample_rows=M, flush=True,
                    h2d=3 * E, d2h=2 * E, dtype="c64", launches=2, kernel="diag_scan_kernel<float2, const, adjoint> (b200_diag_bwd)",
                    fwd=lambda: diagonal_b200.forward(lam, v, x0), bwd=lambda o: diagonal_b200.backward(g, lam, o, x0),
                    e2e=e2e, cpu=cpu)
    if name == "C3":
        Bn, L, D, N = 32, 2048, 512, 16
        draw = rn(Bn, L, D) * 0.5 - 3.0
        A = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).expand(D, N).contiguous()
        Bt, Ct, u, z, gout = rn(Bn, L, N), rn(Bn, L, N), rn(Bn, L, D), rn(Bn, L, D), rn(Bn, L, D)
        Dp = torch.ones(D, device=dev)
        ins = (draw, A, Bt, Ct, u, z, Dp, None)
        big, small = Bn * L * D * 4, Bn * L * N * 4
        hin = [pin(t) for t in (draw, Bt, Ct, u, z, gout)]
        hout = [pin(draw) for _ in range(4)] + [pin(Bt), pin(Bt)] if host_buffers else []

        def e2e():
            d_, b_, c_, u_, z_, g_ = (t.to(dev, non_blocking=True) for t in hin)
            leaves = [t.requires_grad_() for t in (d_, b_, c_, u_, z_)]
            A_, Dp_ = A.clone().requires_grad_(), Dp.clone().requires_grad_()
            out, _ = mamba_b200.run(leaves[0], A_, leaves[1], leaves[2], leaves[3], leaves[4], Dp_, None)
            out.backward(g_)
            for h_, t in zip(hout, (out.detach(), d_.grad, u_.grad, z_.grad, b_.grad, c_.grad)):
                h_.copy_(t, non_blocking=True)
            return A_.grad.cpu()

        def cpu(rows):
            from oracle import oracle as O
            a = [t[:rows].cpu().numpy() if t is not None and t.dim() == 3 else (None if t is None else t.cpu().numpy()) for t in ins]
            go = gout[:rows].cpu().numpy()
            return lambda: (O.mamba_fwd(*a), O.mamba_bwd(*a, go, None))

        def ref_cpu(rows):  # tsfast's C kernel for the fused section (architectures/mamba/backend_c.py)
            _import_reference()
            from tsfast.models.architectures.mamba import backend_c

            host = [None if t is None else (t[:rows].cpu() if t.dim() == 3 else t.cpu()) for t in ins]
            go = gout[:rows].cpu()
            why = backend_c.supports(*host)
            if why is not None:
                raise RuntimeError(why)

            def one():
                leaves = [None if t is None else t.clone().requires_grad_() for t in host]
                out, _ = backend_c.run(*leaves)
                out.backward(go)
            return one, "mamba.backend_c.run (tsfast's C kernel for the fused selective-scan section)"

        return dict(desc="C3: Mamba selective scan fwd+bwd, B=32 T=2048 D_inner=512 N=16 fp32, S4D-real A, D=1, SiLU gate",
                    ref_cpu=ref_cpu, fwd_bytes=4 * big + 2 * small + Bn * D * N * 4, bwd_bytes=7 * big + 4 * small,
                    elems=2 * Bn * L * D * N, rows=Bn, sample_rows=2, flush=False, h2d=4 * big + 2 * small + big,
                    d2h=4 * big + 2 * small, dtype="f32", launches=6, kernel="mamba_bwd_kernel<TPC=4> (b200_mamba_bwd)",
                    traffic=815_733_248 + 499_814_144,  # ncu dram__bytes read + write of one adjoint launch at this shape
                    fwd=lambda: mamba_b200._scan_train_op(*ins), bwd=lambda o: mamba_b200._scan_bwd_op(gout, None, o[2], *ins),
                    e2e=e2e, cpu=cpu)
    if name == "C4":
        P, Bn, L = 128, 128, 8192
        rng = np.random.default_rng(1234 + rank)
        a0 = np.zeros((P, 4))
        for i in range(P):
            poles = []
            for _ in range(2):
                rr, th = rng.uniform(0.5, 0.95), rng.uniform(0, np.pi)
                poles += [rr * np.exp(1j * th), rr * np.exp(-1j * th)]
            a0[i] = np.real(np.poly(poles))[1:]
        a_p = torch.from_numpy(a0.astype(np.float32)).to(dev)
        a = a_p.expand(Bn, P, 4).reshape(-1, 4).contiguous()
        w, g = rn(Bn * P, L), rn(Bn * P, L)
        E = Bn * P * L * 4
        hw, hg, hy, hgw = pin(w), pin(g), pin(w), pin(w)

        def e2e():
            dw = hw.to(dev, non_blocking=True).view(Bn, P, L).requires_grad_()
            ap = a_p.clone().requires_grad_()
            y = allpole_b200.run(ap, dw, None)
            y.backward(hg.to(dev, non_blocking=True).view(Bn, P, L))
            hy.copy_(y.detach().view(-1, L), non_blocking=True)
            hgw.copy_(dw.grad.view(-1, L), non_blocking=True)
            return ap.grad.cpu()

        def cpu(rows):
            from oracle import oracle as O
            a_, w_, g_ = a[: rows * P].cpu().numpy(), w[: rows * P].cpu().numpy(), g[: rows * P].cpu().numpy()
            return lambda: O.allpole_bwd(g_, a_, O.allpole_fwd(a_, w_, None), None)

        def ref_cpu(rows):  # tsfast's only CPU path for the all-pole filter: the companion-matrix doubling scan
            _import_reference()
            import torch.nn.functional as F
            from tsfast.models.architectures.dynonet.core import linear_recurrence

            ac = a_p.cpu()
            shift = torch.eye(4)[:-1].expand(P, 3, 4)
            w_, g_ = w[: rows * P].cpu().view(rows, P, L), g[: rows * P].cpu().view(rows, P, L)

            def one():
                aq, wq = ac.clone().requires_grad_(), w_.clone().requires_grad_()
                comp = torch.cat((-aq.unsqueeze(1), shift), dim=1)  # dynonet/core.py:186-190
                x = linear_recurrence(comp, F.pad(wq.unsqueeze(-1), (0, 3)), None)
                x[..., 0].backward(g_)
            return one, "linear_recurrence over the companion form (dynonet/core.py:103-141, 231), tsfast's CPU path for S4"

        return dict(desc="C4: dynoNet all-pole IIR scan fwd+bwd, B=128 x 128 channels, T=8192 fp32, order 4", ref_cpu=ref_cpu,
                    ref_rows=1, fwd_bytes=2 * E, bwd_bytes=3 * E, elems=2 * Bn * P * L, rows=Bn, sample_rows=8, flush=False,
                    h2d=2 * E, d2h=2 * E, dtype="f32", launches=2, kernel="allpole_kernel<NA=4, adjoint> (b200_allpole_bwd)",
                    traffic=1_074_100_000 + 501_500_000,  # ncu dram__bytes read + write of one adjoint launch at this shape
                    fwd=lambda: allpole_b200._allpole_op(a, w, None), bwd=lambda o: allpole_b200._allpole_bwd_op(g, a, o, None),
                    e2e=e2e, cpu=cpu)
    if name == "V":
        from tsfast_b200 import conv_b200

        Bn, L, D, K = 32, 2048, 512, 4
        x, gy, tail = rn(Bn, L, D), rn(Bn, L, D), rn(Bn, D, K - 1)
        w, bias = rn(D, K) * 0.5, rn(D)
        E = Bn * L * D * 4
        hx, hgy, hy, hgx = pin(x), pin(gy), pin(x), pin(x)

        def e2e():
            dx = hx.to(dev, non_blocking=True).requires_grad_()
            ww, bb = w.clone().requires_grad_(), bias.clone().requires_grad_()
            y = conv_b200.run(dx, tail, ww.unsqueeze(1), bb)
            y.backward(hgy.to(dev, non_blocking=True))
            hy.copy_(y.detach(), non_blocking=True)
            hgx.copy_(dx.grad, non_blocking=True)
            return ww.grad.cpu()

        def cpu(rows):
            from oracle import oracle as O_
            x_, g_, t_ = x[:rows].cpu().numpy(), gy[:rows].cpu().numpy(), tail[:rows].cpu().numpy()
            w_, b_ = w.cpu().numpy(), bias.cpu().numpy()
            return lambda: (O_.conv_fwd(x_, t_, w_, b_), O_.conv_bwd(g_, x_, t_, w_, b_))

        return dict(desc="V: Mamba causal depthwise conv (K=4) + SiLU fwd+bwd, B=32 T=2048 D=512 fp32 (the step feeding C3)",
                    fwd_bytes=2 * E, bwd_bytes=3 * E, elems=2 * Bn * L * D, rows=Bn, sample_rows=8, flush=False,
                    h2d=2 * E, d2h=2 * E, dtype="f32", launches=4, kernel="conv_silu_bwd_kernel<K=4> + partial sums (b200_conv_silu_bwd)",
                    traffic=286_489_088 + 96_544_000,  # ncu dram__bytes read + write of one adjoint launch at this shape
                    fwd=lambda: conv_b200._conv_silu_op(x, tail, w, bias),
                    bwd=lambda o: conv_b200._conv_silu_bwd_op(gy, x, tail, w, bias), e2e=e2e, cpu=cpu)
    if name == "P":
        from tsfast_b200 import proj_b200

        # the in-projection of one DeepLRU layer of C5: 128 windows x 2000 steps, 128 features -> 256 complex states
        Mt, K_, N_ = 256000, 128, 512
        a_ = rn(Mt, K_)
        w_ = rn(N_, K_) / K_**0.5
        g_ = rn(Mt, N_)
        big, small = Mt * N_ * 4, Mt * K_ * 4
        ha, hg, hy, hga = pin(a_), pin(g_), pin(g_), pin(a_)

        def e2e():
            da = ha.to(dev, non_blocking=True).requires_grad_()
            ww = w_.clone().requires_grad_()
            y = proj_b200.linear(da, ww)
            y.backward(hg.to(dev, non_blocking=True))
            hy.copy_(y.detach(), non_blocking=True)
            hga.copy_(da.grad, non_blocking=True)
            return ww.grad.cpu()

        def cpu(rows):
            import numpy as np_

            an, wn, gn = a_[: rows * 2000].cpu().numpy(), w_.cpu().numpy(), g_[: rows * 2000].cpu().numpy()
            return lambda: (an @ wn.T, gn @ wn, gn.T @ an)

        def extra(timed):
            wt = w_.t().contiguous()
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = False
            a_ @ wt  # the first call of each mode picks its cuBLAS algorithm
            f32 = timed(lambda: a_ @ wt, 5)
            torch.backends.cuda.matmul.allow_tf32 = True
            a_ @ wt
            tf32 = timed(lambda: a_ @ wt, 5)
            torch.backends.cuda.matmul.allow_tf32 = prev
            return {"forward_pytorch_float32_ms": round(f32, 4), "forward_pytorch_tf32_ms": round(tf32, 4),
                    "flops_per_step": 3 * 2 * Mt * K_ * N_, "arithmetic": "tcgen05.mma.kind::tf32, 3 MMAs per product (hi/lo split)"}

        return dict(desc="P: LRU in-projection GEMM of C5, 256000 tokens x 128 features -> 512 (256 complex states) fp32, "
                         "forward + input gradient + weight gradient",
                    fwd_bytes=big + small, bwd_bytes=2 * (big + small), elems=Mt * N_, rows=128, sample_rows=8, flush=False,
                    h2d=big + small, d2h=big + small, dtype="f32 (tf32 x3)", launches=6,
                    kernel="proj_gemm_ws_kernel + proj_wgrad_ws_kernel (b200_proj_gemm, b200_proj_wgrad)",
                    fwd=lambda: proj_b200._proj_gemm_op(a_, w_, None),
                    bwd=lambda o: (proj_b200._input_grad(g_, w_), proj_b200._proj_wgrad_op(g_, a_)), e2e=e2e, cpu=cpu, extra=extra)
    if name == "G":
        from tsfast_b200 import dynonet_b200

        Bn, L, I, O, nb, na = 128, 8192, 8, 16, 8, 4
        P = I * O
        rng = np.random.default_rng(4321 + rank)
        a0 = np.zeros((O, I, na))
        for i in range(O):
            for j in range(I):
                poles = []
                for _ in range(2):
                    rr, th = rng.uniform(0.5, 0.95), rng.uniform(0, np.pi)
                    poles += [rr * np.exp(1j * th), rr * np.exp(-1j * th)]
                a0[i, j] = np.real(np.poly(poles))[1:]
        a_c = torch.from_numpy(a0.astype(np.float32)).to(dev).requires_grad_()
        b_c = (rn(O, I, nb) * 0.3).requires_grad_()
        u = rn(Bn, L, I).requires_grad_()
        gy = rn(Bn, L, O)
        hu, hgy, hy, hgu = pin(u.detach()), pin(gy), pin(gy), pin(u.detach())

        def fwd():
            return dynonet_b200.linear_block(u, b_c, a_c, None)[0]

        def bwd(y):
            return torch.autograd.grad(y, (u, b_c, a_c), gy, retain_graph=True)  # timed repeatedly on one graph

        def unfused():  # the reference's formulation with this package's all-pole op in the middle
            import torch.nn.functional as F
            with torch.no_grad():
                u_buf = torch.cat((u.new_zeros(Bn, nb - 1, I), u), 1)
                weight = b_c.permute(1, 0, 2).reshape(P, 1, nb).flip(-1)
                w_ = F.conv1d(u_buf.transpose(1, 2), weight, groups=I)
                yp = allpole_b200.run(a_c.permute(1, 0, 2).reshape(P, na), w_, None)
                return yp.view(Bn, I, O, L).sum(1).transpose(1, 2)

        def extra(timed):
            unfused()  # the first grouped conv1d call picks its algorithm
            with torch.no_grad():
                fused_ms = timed(lambda: dynonet_b200.linear_block(u, b_c, a_c, None), 5)
            return {"forward_no_grad_ms": round(fused_ms, 4), "forward_unfused_ms": round(timed(unfused, 5), 4),
                    "unfused": "grouped conv1d + b200 all-pole op + sum over inputs, as dynonet/core.py:214-250"}

        def e2e():
            du = hu.to(dev, non_blocking=True).requires_grad_()
            bb, aa = b_c.detach().clone().requires_grad_(), a_c.detach().clone().requires_grad_()
            y = dynonet_b200.linear_block(du, bb, aa, None)[0]
            y.backward(hgy.to(dev, non_blocking=True))
            hy.copy_(y.detach(), non_blocking=True)
            hgu.copy_(du.grad, non_blocking=True)
            return bb.grad.cpu()

        def cpu(rows):
            from oracle import oracle as O_
            u_, g_ = u.detach()[:rows].cpu().numpy(), gy[:rows].cpu().numpy()
            b_, a_ = b_c.detach().cpu().numpy(), a_c.detach().cpu().numpy()

            def run():
                y, yp, _, _ = O_.gblock_fwd(u_, b_, a_)
                return O_.gblock_bwd(g_, u_, b_, a_, yp)
            return run

        E = Bn * L * 4
        return dict(desc="G: dynoNet G-block (FIR nb=8 + all-pole na=4 + sum over inputs) training step, B=128 T=8192, "
                         "8 inputs x 16 outputs = 128 filters, fp32",
                    fwd_bytes=E * (I + O + P), bwd_bytes=E * (O + P + 2 * I), elems=2 * Bn * P * L, rows=Bn, sample_rows=2,
                    flush=False, h2d=E * (I + O), d2h=E * (I + O), dtype="f32", launches=3,
                    kernel="allpole_kernel<NA=4, adjoint, row map> + gblock_num_bwd_kernel (b200_gblock_bwd)",
                    fwd=fwd, bwd=bwd, e2e=e2e, cpu=cpu, extra=extra)
    raise SystemExit(f"unknown workload {name}")


def run_workload(args):
    torch, dist, world, rank, local, dev, barrier = _dist_setup()
    if args.workload == "C5":
        return _run_c5(args, torch, dist, dev, world, rank, local, barrier)
    wl = _workload(args.workload, torch, dev, rank)
    timed = _make_timed(torch, dev)
    keep = {}

    def step():
        keep["o"] = wl["fwd"]()
        wl["bwd"](keep["o"])

    for _ in range(args.warmup):
        step()
    barrier()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    ms = timed(step, args.steps)
    barrier()
    clock_rec = clocks.stop() if rank == 0 else None
    n = max(3, min(args.steps, 10))
    fwd_ms = timed(lambda: keep.__setitem__("o", wl["fwd"]()), n)
    bwd_ms = timed(lambda: wl["bwd"](keep["o"]), n)
    e2e_ms = float("nan")
    if not args.kernel_only:
        wl["e2e"]()
        barrier()
        e2e_ms = timed(wl["e2e"], max(2, min(args.steps, 5)))
    times = torch.tensor([ms, e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(x) for x in times.tolist())
    if rank == 0:
        peak, peak_src = _peaks()
        step_bytes = wl["fwd_bytes"] + wl["bwd_bytes"]
        base = None
        if world == 1 and not args.no_cpu and not args.kernel_only:
            from oracle import oracle as O
            O.build()
            O.set_num_threads(_host_threads())
            base, why = None, "no reference leg for this workload"
            if "ref_cpu" in wl:  # the reference's own CPU implementation, from the copy under oracle/_ref
                base, why = _reference_cpu_leg(wl, torch, 10.0)
            if base is None:
                rows = wl["sample_rows"]
                sec, cnt = _time_cpu(wl["cpu"](rows), 1, 1, 10.0)
                base = {"value": round(step_bytes * rows / wl["rows"] / sec / 1e9, 3), "unit": "GB/s", "cores": O.num_threads(),
                        "kind": "port", "sample": f"{rows} of {wl['rows']} batch rows, fwd+bwd, median of {cnt} passes of "
                        f"{sec * 1e3:.1f} ms; float32 C port of the reference's CPU algorithm, OpenMP ({why})"}
        bwd_gbs, fwd_gbs = wl["bwd_bytes"] / bwd_ms / 1e6, wl["fwd_bytes"] / fwd_ms / 1e6
        extra = wl["extra"](timed) if "extra" in wl else {}
        _emit({
            "metric": METRIC, "value": round(step_bytes * world / ms / 1e6, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": wl["desc"], "algorithmic_bytes_per_step_per_gpu": step_bytes,
                       "state_elements_per_s": round(wl["elems"] * world / (ms * 1e-3)),
                       "l2": ("working set fits in L2; " if wl["flush"] else "streamed tensors are larger than the 126 MB L2; ")
                             + "a 256 MB buffer is rewritten before every timed call",
                       "timing": "CUDA events around every step (enqueued behind an L2-flushing write so that host launch time is not inside), averaged", "sharding": "independent sequences per rank, no collective",
                       **extra},
            "roofline": {"bound": "hbm", "kernel": wl["kernel"], "achieved": round(bwd_gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(bwd_gbs / peak, 4), "traffic": wl.get("traffic"), "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": wl["bwd_bytes"], "ms_per_launch": round(bwd_ms, 4),
                         "forward_kernel": {"achieved": round(fwd_gbs, 1), "frac": round(fwd_gbs / peak, 4),
                                            "algorithmic_bytes_per_launch": wl["fwd_bytes"], "ms_per_launch": round(fwd_ms, 4)}},
            "cpu_baseline": base,
            "e2e": None if args.kernel_only else {"value": round(step_bytes * world / e2e_ms / 1e6, 2), "unit": "GB/s",
                                                  "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"],
                                                  "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": wl["launches"] * args.steps, "clocks": clock_rec})
    if world > 1:
        dist.destroy_process_group()


C5_SHAPE = dict(windows=128, T=2000, d_model=128, d_state=256, n_layers=4)


def _c5_setup(torch, dev, rank, plain_gemms=False):
    """C5: DeepLRU (1 in, 1 out, 4 blocks, width 128, 256 complex states), 128 windows of T=2000 per
    GPU: band-limited Gaussian noise in (sigma 0.1, cut-off 0.4 Nyquist), a seeded stable 2nd-order
    filter followed by tanh as target.  Replicas start identical (same seed on every rank)."""
    import numpy as np
    from scipy import signal

    import tsfast_b200

    # the caller is tsfast's own DeepLRU (unmodified copy under oracle/_ref); install() routes its
    # diagonal scans to this package's kernels, which is how a tsfast user runs them
    _import_reference()
    from tsfast.models import DeepLRU

    tsfast_b200.uninstall()
    tsfast_b200.install(fuse_projections=not plain_gemms)
    Bn, T_, dm, ds, nl = (C5_SHAPE[k] for k in ("windows", "T", "d_model", "d_state", "n_layers"))
    rng = np.random.default_rng(100 + rank)
    bl, al = signal.butter(4, 0.4)
    x_np = signal.lfilter(bl, al, rng.standard_normal((Bn, T_ + 200)), axis=1)[:, 200:]
    x_np = 0.1 * x_np / x_np.std()
    sys_rng = np.random.default_rng(7)  # the plant is the same on every rank
    pr, pth = sys_rng.uniform(0.7, 0.95), sys_rng.uniform(0.1, 0.6)
    den = [1.0, -2 * pr * np.cos(pth), pr * pr]
    y_np = np.tanh(signal.lfilter([sum(den)], den, x_np, axis=1) * 5.0)
    hx = torch.from_numpy(x_np.astype(np.float32)).unsqueeze(-1).pin_memory()
    hy = torch.from_numpy(y_np.astype(np.float32)).unsqueeze(-1).pin_memory()
    torch.manual_seed(0)
    model = DeepLRU(1, 1, d_model=dm, d_state=ds, n_layers=nl, r_min=0.0, r_max=1.0).to(dev)
    if not plain_gemms:  # boundary projections (install above) and every nn.Linear on the tcgen05 GEMM
        tsfast_b200.accelerate_linears(model)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    return model, opt, hx, hy


def _c5_step_fn(torch, model, opt, ar_events):
    from tsfast_b200.dist import allreduce_gradients

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        allreduce_gradients(model.parameters(), average=True)
        a1.record()
        opt.step()
        ar_events.append((a0, a1))
        return loss

    return step


def _c5_measure(torch, dist, dev, world, rank, local, barrier, steps, warmup, plain_gemms=False):
    """`steps` DeepLRU training steps (forward, MSE, backward, one flat-bucket NCCL all-reduce of the
    gradients, Adam) between two events; this rank's time (the caller takes the max over ranks).
    `plain_gemms` leaves the model's GEMMs to PyTorch (float32 cuBLAS) for comparison."""
    model, opt, hx, hy = _c5_setup(torch, dev, rank, plain_gemms)
    xb, yb = hx.to(dev), hy.to(dev)
    ar = []
    step = _c5_step_fn(torch, model, opt, ar)
    for _ in range(warmup):
        step(xb, yb)
    barrier()
    ar.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step(xb, yb)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    return {"workload": "C5: DeepLRU(1,1,d_model=128,d_state=256,n_layers=4) training step, 128 windows of T=2000 per GPU "
                        f"({C5_SHAPE['windows'] * world} global), Adam, NCCL gradient all-reduce",
            "ms_per_step": round(ms, 3), "steps": steps, "windows_per_gpu": C5_SHAPE["windows"],
            "windows_per_s": round(C5_SHAPE["windows"] * world / (ms * 1e-3), 1),
            "allreduce_ms": round(statistics.mean(a.elapsed_time(b) for a, b in ar), 3), "final_loss": round(float(loss.detach()), 6)}


def _run_c5(args, torch, dist, dev, world, rank, local, barrier):
    """`--workload C5`: the full line for the DeepLRU step.  `value` counts the algorithmic bytes of
    the eight scan passes (4 blocks x (2 + 3) complex tensors of 524 MB) per step time; the scan
    kernels are also timed alone at the layer shape."""
    from tsfast_b200.scan_backends import diagonal_b200

    Bn, T_, ds, nl = C5_SHAPE["windows"], C5_SHAPE["T"], C5_SHAPE["d_state"], C5_SHAPE["n_layers"]
    model, opt, hx, hy = _c5_setup(torch, dev, rank)
    xb, yb = hx.to(dev), hy.to(dev)
    n_params = sum(p.numel() for p in model.parameters())
    ar_ms = []
    step = _c5_step_fn(torch, model, opt, ar_ms)

    for _ in range(args.warmup):
        step(xb, yb)
    barrier()
    ar_ms.clear()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from tsfast_b200 import glue_b200, proj_b200

    def lib_calls():  # calls into the library so far: scans, projection GEMMs / weight gradients, block glue
        return diagonal_b200.calls + proj_b200.calls + glue_b200.calls

    barrier()
    calls0 = lib_calls()
    e0.record()
    for _ in range(args.steps):
        loss = step(xb, yb)
    e1.record()
    barrier()
    launches = lib_calls() - calls0
    ms = e0.elapsed_time(e1) / args.steps
    clock_rec = clocks.stop() if rank == 0 else None
    allreduce_ms = statistics.mean(a.elapsed_time(b) for a, b in ar_ms)

    # end to end: the batch comes from pinned host memory every step, the loss goes back
    e2e_steps = max(2, min(args.steps, 5))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(e2e_steps):
        lval = step(hx.to(dev, non_blocking=True), hy.to(dev, non_blocking=True)).item()
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1) / e2e_steps

    # the scan kernels alone at the layer shape (complex64, M=128, L=2000, N=256)
    lru = model.blocks[0].lru
    lam = torch.polar(torch.exp(-torch.exp(lru.nu_log)), torch.exp(lru.theta_log)).detach().expand(Bn, ds).contiguous()
    v = torch.randn(Bn, T_, ds, device=dev, dtype=torch.complex64)
    g = torch.randn(Bn, T_, ds, device=dev, dtype=torch.complex64)
    out = diagonal_b200.forward(lam, v, None)
    k0, k1, k2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    torch.cuda.synchronize()
    k0.record()
    for _ in range(5):
        out = diagonal_b200.forward(lam, v, None)
    k1.record()
    for _ in range(5):
        diagonal_b200.backward(g, lam, out, None)
    k2.record()
    torch.cuda.synchronize()
    fwd_ms, bwd_ms = k0.elapsed_time(k1) / 5, k1.elapsed_time(k2) / 5

    times = torch.tensor([ms, e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(x) for x in times.tolist())
    if rank == 0:
        peak, peak_src = _peaks()
        E = Bn * T_ * ds * 8
        scan_bytes = nl * 5 * E
        bwd_gbs, fwd_gbs = 3 * E / bwd_ms / 1e6, 2 * E / fwd_ms / 1e6
        _emit({
            "metric": METRIC, "value": round(scan_bytes * world / ms / 1e6, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "c64", "data": "synthetic",
            "config": {"workload": "C5: DeepLRU(1,1,d_model=128,d_state=256,n_layers=4) training step, "
                                   f"{Bn} windows of T={T_} per GPU ({Bn * world} global), Adam, NCCL gradient all-reduce",
                       "algorithmic_scan_bytes_per_step_per_gpu": scan_bytes, "windows_per_s": round(Bn * world / (ms * 1e-3), 1),
                       "parameters": n_params, "allreduce_ms": round(allreduce_ms, 3),
                       "scan_share_of_step": round(nl * (fwd_ms + bwd_ms) / ms, 3), "final_loss": round(float(lval), 6),
                       "l2": "every scan tensor is 524 MB, larger than L2; no flush needed",
                       "note": "value counts scan bytes only; the step also runs the projections, norms and GLU"},
            "roofline": {"bound": "hbm", "kernel": "diag_stream_kernel<float2, const, adjoint> (b200_diag_bwd)",
                         "achieved": round(bwd_gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(bwd_gbs / peak, 4),
                         "traffic": None, "peak_source": peak_src, "algorithmic_bytes_per_launch": 3 * E,
                         "ms_per_launch": round(bwd_ms, 4),
                         "forward_kernel": {"achieved": round(fwd_gbs, 1), "frac": round(fwd_gbs / peak, 4),
                                            "algorithmic_bytes_per_launch": 2 * E, "ms_per_launch": round(fwd_ms, 4)}},
            "cpu_baseline": None,
            "e2e": {"value": round(scan_bytes * world / e2e_ms / 1e6, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": 2 * Bn * T_ * 4, "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": launches, "clocks": clock_rec})
    if world > 1:
        dist.destroy_process_group()


def _fail_line(exc: BaseException) -> dict:
    """One line that names the rank, the error and the innermost frame of this file it came from."""
    where = "?"
    for fr in reversed(traceback.extract_tb(exc.__traceback__)):
        if Path(fr.filename).name == Path(__file__).name:
            where = f"{fr.name}:{fr.lineno}"
            break
    return {"rank": int(os.environ.get("RANK", "0")), "error": f"{type(exc).__name__}: {exc}"[:600], "where": where}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=["C1", "C2", "C3", "C4", "C5", "G", "V", "P"], default="C2")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-triton", action="store_true", help="skip the reference's Triton kernels (single-GPU baseline leg)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (no end-to-end, CPU or extra-workload legs): the command profiled under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    try:
        if args.impl == "reference":
            run_reference(args)
        elif args.workload == "C2":
            run_gpu(args)
        else:
            run_workload(args)
    except BaseException as exc:  # every rank says why it dies, on one line, on both streams
        if isinstance(exc, SystemExit) and exc.code in (0, None):
            raise
        text = json.dumps(_fail_line(exc))
        print(text, flush=True)
        print(text, file=sys.stderr, flush=True)
        traceback.print_exc()
        raise SystemExit(1)


try:  # under torchrun, also hand the traceback to the elastic agent's error file
    from torch.distributed.elastic.multiprocessing.errors import record as _record

    main = _record(main)
except Exception:  # pragma: no cover - torch without the elastic package
    pass


if __name__ == "__main__":
    main()
