#!/usr/bin/env python3
"""Benchmark of the sm_100a op library (see DESIGN.md for what each number means).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload auto|elementwise|mlp]
    python bench.py --impl reference ...      # the CPU arm: the oracle port on the host cores

One JSON line is printed by rank 0.  `value` is whole-job throughput with inputs resident
in HBM; `e2e` is the same metric through the C ABI with host buffers (copies inside the
timed region); `roofline` describes the dominant kernel; `cpu_baseline` is the CPU port of
the reference's backend timed on this box; `sweeps` lists every single-op case with its
achieved HBM GB/s.  torch is used for device memory, events and (N > 1) torch.distributed;
every op in the timed regions is a call into libmaidenx_cuda.so.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from maidenx_b200 import sweeps  # noqa: E402

SZ = ctypes.c_size_t
NOMINAL_HBM_GBS = 8000.0          # the figure the target configuration quotes (~8 TB/s)
FALLBACK_HBM_GBS = 6650.0         # used only when MEASURED_PEAKS.json is absent
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(sm)[len(sm) // 2:]  # upper half: samples taken under load
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# op launching through the C ABI
# ---------------------------------------------------------------------------------------
class Launcher:
    """Binds the entry point of a sweep case to device buffers; `launch()` is exactly one
    call of cuda_<op>_<dtype> with a host-resident metadata block."""

    def __init__(self, lib_mod, case, bufs):
        self.case = case
        self.fn = lib_mod.op(case.op, case.dtype)
        self.meta = np.asarray(case.metadata, dtype=np.uint64)
        m = self.meta.ctypes.data
        c = case
        if c.family == "binary":
            self.args = (SZ(c.num_els), SZ(2), m, bufs["a"], bufs["b"], bufs["out"])
        elif c.family == "unary":
            self.args = (SZ(c.num_els), SZ(2), m, bufs["a"], bufs["out"])
        elif c.family == "reduce":
            self.args = (SZ(c.num_els), SZ(2), SZ(c.extra["num_red"]), m, bufs["a"], bufs["out"])
        elif c.family == "sum_to_shape":
            self.args = (SZ(c.num_els), SZ(3), m, bufs["a"], bufs["out"])
        elif c.family in ("im2col", "col2im"):
            self.args = (SZ(c.num_els), m, bufs["a"], bufs["out"])
        else:
            raise KeyError(c.family)

    def launch(self):
        self.fn(*self.args)


TORCH_DT = None


def torch_dtype(name):
    import torch
    return {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "i32": torch.int32}[name]


def make_inputs(torch, dtype, count, seed, dist="uniform"):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    if dtype == "i32":
        return torch.randint(-1000, 1001, (count,), dtype=torch.int32, device="cuda", generator=g)
    if dist == "normal":
        x = torch.randn(count, device="cuda", generator=g)
    else:
        x = torch.rand(count, device="cuda", generator=g) * 2 - 1
    return x.to(torch_dtype(dtype))


def time_launches(torch, fn, iters, warm):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters  # ms per launch


KERNEL_OF_LAYOUT = {"contiguous": "ew_flat_kernel", "transposed_lhs": "ew_tile_kernel", "transposed": "ew_tile_kernel",
                    "rhs_broadcast": "ew_row_long_kernel", "broadcast": "ew_row_long_kernel"}


def run_sweep_group(torch, lib_mod, cases, iters, warm, seeds, dist):
    """Per-case device timing.  Inputs are allocated per dtype once and are larger than L2
    (or stream through it: the smallest working set is 3x the 126 MB L2)."""
    rows = []
    by_dtype = {}
    for c in cases:
        by_dtype.setdefault(c.dtype, []).append(c)
    for dt, cs in by_dtype.items():
        na = max(c.in_elems[0] for c in cs)
        nb = max((c.in_elems[1] for c in cs if len(c.in_elems) > 1), default=0)
        no = max(c.out_elems for c in cs)
        a = make_inputs(torch, dt, na, seeds[0], dist)
        b = make_inputs(torch, dt, nb, seeds[1], dist) if nb else None
        if dt != "i32" and b is not None:
            b = torch.where(b == 0, torch.ones_like(b), b)  # keep div on its arithmetic path
        out = torch.empty(no, dtype=torch_dtype(dt), device="cuda")
        bufs = {"a": a.data_ptr(), "b": b.data_ptr() if b is not None else None, "out": out.data_ptr()}
        for c in cs:
            L = Launcher(lib_mod, c, bufs)
            ms = time_launches(torch, L.launch, iters, warm)
            rows.append({"case": c.name, "ms": round(ms, 4), "gbs": round(c.bytes / ms / 1e6, 1), "bytes": c.bytes})
        del a, b, out
        torch.cuda.empty_cache()
    return rows


# ---------------------------------------------------------------------------------------
# workload: elementwise sweep (the headline single-GPU configuration)
# ---------------------------------------------------------------------------------------
def elementwise_workload(torch, lib_mod, args, rank, world):
    cases = sweeps.elementwise_cases()
    # device-resident inputs per dtype
    state = {}
    for dt in ("f32", "bf16", "f16", "i32"):
        n = 16384 * 16384
        a = make_inputs(torch, dt, n, 1 if dt != "i32" else 2)
        b = make_inputs(torch, dt, n, 101 if dt != "i32" else 102)
        if dt != "i32":
            b = torch.where(b == 0, torch.ones_like(b), b)
        out = torch.empty(n, dtype=torch_dtype(dt), device="cuda")
        state[dt] = (a, b, out)
    launchers = []
    for c in cases:
        a, b, out = state[c.dtype]
        launchers.append(Launcher(lib_mod, c, {"a": a.data_ptr(), "b": b.data_ptr(), "out": out.data_ptr()}))
    step_bytes = sum(c.bytes for c in cases)

    def step():
        for L in launchers:
            L.launch()

    return {"name": "strided elementwise sweep, 2^28-element tensors [16384,16384], f32/bf16/f16 + i32",
            "step": step, "units_per_step": step_bytes / 1e9, "launches_per_step": len(launchers), "cases": cases,
            "launchers": launchers, "state": state, "metric": "elementwise_hbm_throughput", "unit": "GB/s", "dtype": "f32/bf16/f16/i32"}


def e2e_elementwise(torch, lib_mod, wl, steps, warm):
    """Same sweep through the C ABI with host buffers: cuda_memcpy_h2d of each case's
    inputs from pinned memory, the op, cuda_memcpy_d2h of its output, all timed."""
    lib = lib_mod.load()
    pinned = {}
    for dt, (a, b, out) in wl["state"].items():
        pinned[dt] = (a.cpu().pin_memory(), b.cpu().pin_memory(), torch.empty(out.shape, dtype=out.dtype).pin_memory())
    h2d = d2h = 0
    plan = []
    for c, L in zip(wl["cases"], wl["launchers"]):
        a, b, out = wl["state"][c.dtype]
        ha, hb, ho = pinned[c.dtype]
        es = a.element_size()
        copies = [(a.data_ptr(), ha.data_ptr(), c.in_elems[0] * es)]
        if len(c.in_elems) > 1:
            copies.append((b.data_ptr(), hb.data_ptr(), c.in_elems[1] * es))
        plan.append((L, copies, (ho.data_ptr(), out.data_ptr(), c.out_elems * es)))
        h2d += sum(x[2] for x in copies)
        d2h += c.out_elems * es

    def step():
        for L, copies, (hdst, dsrc, nbytes) in plan:
            for ddst, hsrc, nb in copies:
                lib.cuda_memcpy_h2d(ddst, hsrc, nb)
            L.launch()
            lib.cuda_memcpy_d2h(hdst, dsrc, nbytes)

    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    dt_s = (time.perf_counter() - t0) / steps
    return {"value": round(wl["units_per_step"] / dt_s, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "note": "every case copies its inputs host->device and its output device->host through cuda_memcpy_*"}


# ---------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU backend on the host cores
# ---------------------------------------------------------------------------------------
def cpu_sweep(cases_fn, R, C, passes):
    """Times the oracle on a bounded sample: the same sweep at [R, C] instead of [16384, 16384]."""
    from oracle import binding
    binding.load()
    binding.set_reduce_parallel(True)
    threads = binding.max_threads()
    cases = cases_fn(R, C)
    rng = np.random.default_rng(1)
    npdt = {"f32": np.float32, "bf16": np.uint16, "f16": np.float16, "i32": np.int32}
    from maidenx_b200 import dtypes as D
    bufs = {}
    for dt in {c.dtype for c in cases}:
        n = R * C
        if dt == "i32":
            a, b = rng.integers(-1000, 1001, n).astype(np.int32), rng.integers(-1000, 1001, n).astype(np.int32)
        else:
            a = D.encode(rng.uniform(-1, 1, n).astype(np.float32), D.BY_NAME[dt])
            b = D.encode(rng.uniform(0.1, 1, n).astype(np.float32), D.BY_NAME[dt])
        bufs[dt] = (a, b, np.empty(n, dtype=npdt[dt]))
    calls = []
    for c in cases:
        a, b, out = bufs[c.dtype]
        m = np.asarray(c.metadata, dtype=np.uint64)
        fn = binding.op(c.op, c.dtype)
        if c.family == "binary":
            calls.append((fn, (SZ(c.num_els), SZ(2), m.ctypes.data, a.ctypes.data, b.ctypes.data, out.ctypes.data), m))
        else:
            calls.append((fn, (SZ(c.num_els), SZ(2), m.ctypes.data, a.ctypes.data, out.ctypes.data), m))
    total_bytes = sum(c.bytes for c in cases)
    times = []
    for _ in range(passes):
        t0 = time.perf_counter()
        for fn, a, _ in calls:
            fn(*a)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": round(total_bytes / best / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"the same {len(cases)}-case sweep on [{R},{C}] tensors ({R * C} elements), best of {passes} passes, "
                      f"{best:.2f} s per pass"}, best, total_bytes


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    R = C = 4096
    passes = max(1, args.steps)
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_sweep(sweeps.elementwise_cases, R, C, 1)
    cb, best, total_bytes = cpu_sweep(sweeps.elementwise_cases, R, C, passes)
    line = {"metric": "elementwise_hbm_throughput", "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(best * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32/bf16/f16/i32", "data": "synthetic", "impl": "reference",
            "config": {"workload": "strided elementwise sweep (CPU sample [4096,4096])"},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "elementwise"])
    ap.add_argument("--no-sweeps", action="store_true", help="skip the per-case tables (reductions, conv)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--only-case", default=None, help="profiling aid: launch just this sweep case --steps times and exit")
    ap.add_argument("--small", action="store_true", help="profiling aid: 8192x8192 / quarter-size tensors for ncu captures")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from maidenx_b200 import _lib as lib_mod

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    lib = lib_mod.load()  # raises if the CUDA library is not built: there is no fallback
    assert lib.cuda_set_device(local_rank) == 0
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()

    if args.only_case:
        run_only_case(torch, lib_mod, args)
        return

    args.warmup = max(args.warmup, 3)
    wl = elementwise_workload(torch, lib_mod, args, rank, world)

    sampler = ClockSampler(local_rank)
    for _ in range(args.warmup):
        wl["step"]()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(args.steps):
        wl["step"]()
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_step = s.elapsed_time(e) / args.steps
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms_step], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())
    err = lib.mx_last_error()
    if err:
        raise RuntimeError(f"op library reported status {err} at {lib.mx_last_error_where().decode()}")
    value = wl["units_per_step"] * world / (ms_step / 1e3)

    # per-case tables and the roofline of the dominant kernel (rank 0 only)
    sweeps_out, roofline, e2e, cpu = {}, None, None, None
    if rank == 0:
        rows = []
        for c, L in zip(wl["cases"], wl["launchers"]):
            ms = time_launches(torch, L.launch, max(3, min(args.steps, 10)), 2)
            rows.append({"case": c.name, "ms": round(ms, 4), "gbs": round(c.bytes / ms / 1e6, 1), "bytes": c.bytes})
        sweeps_out["elementwise"] = rows
        by_kernel = {}
        for r in rows:
            k = KERNEL_OF_LAYOUT[r["case"].split("/")[1]]
            t = by_kernel.setdefault(k, [0.0, 0, 0])
            t[0] += r["ms"]
            t[1] += r["bytes"]
            t[2] += 1
        dom = max(by_kernel, key=lambda k: by_kernel[k][0])
        achieved = by_kernel[dom][1] / by_kernel[dom][0] / 1e6
        traffic = None
        tp = ROOT / "profiles" / "ncu_traffic.json"
        if tp.exists():
            ratio = json.loads(tp.read_text()).get(dom, {}).get("dram_bytes_per_algorithmic_byte")
            if ratio:
                traffic = int(ratio * by_kernel[dom][1] / by_kernel[dom][2])
        roofline = {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"], "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                    "launches_timed": by_kernel[dom][2], "traffic": traffic,
                    "share_of_step_time": round(by_kernel[dom][0] / sum(v[0] for v in by_kernel.values()), 3),
                    "per_kernel": {k: {"gbs": round(v[1] / v[0] / 1e6, 1), "frac": round(v[1] / v[0] / 1e6 / peaks["hbm_gbs"], 4)} for k, v in by_kernel.items()}}
        if not args.no_sweeps:
            # free the big elementwise buffers before the other groups allocate theirs
            wl_state = wl.pop("state")
            sweeps_keep = wl_state
            sweeps_out["reduction"] = run_sweep_group(torch, lib_mod, sweeps.reduction_cases(), 10, 3, (3, 103), "normal")
            sweeps_out["conv"] = run_sweep_group(torch, lib_mod, sweeps.conv_cases(), 10, 3, (10, 110), "normal")
            wl["state"] = sweeps_keep
            for grp in ("reduction", "conv"):
                for r in sweeps_out[grp]:
                    r["frac"] = round(r["gbs"] / peaks["hbm_gbs"], 4)
        for r in rows:
            r["frac"] = round(r["gbs"] / peaks["hbm_gbs"], 4)
        if not args.no_e2e:
            e2e = e2e_elementwise(torch, lib_mod, wl, steps=2, warm=1)
        if not args.no_cpu:
            cpu, _, _ = cpu_sweep(sweeps.elementwise_cases, 4096, 4096, 3)
        err = lib.mx_last_error()
        if err:
            raise RuntimeError(f"op library reported status {err} at {lib.mx_last_error_where().decode()}")

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        line = {"metric": wl["metric"], "value": round(value, 2), "unit": wl["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"],
                "data": "synthetic (seeded U(-1,1); i32 U[-1000,1000])",
                "config": {"workload": wl["name"], "l2": "inputs larger than L2 (smallest per-launch working set is 1 GiB vs 126 MB)",
                           "replicas": world},
                "clocks": clocks, "gpu_launches": wl["launches_per_step"] * args.steps, "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu,
                "sweeps": sweeps_out}
        print(json.dumps(line))


def run_only_case(torch, lib_mod, args):
    """Launch one sweep case a few times (for ncu captures of a single kernel)."""
    if args.small:
        groups = sweeps.elementwise_cases(8192, 8192) + sweeps.reduction_cases(4096, 16384, (16, 512, 4096)) + sweeps.conv_cases(N=16)
    else:
        groups = sweeps.elementwise_cases() + sweeps.reduction_cases() + sweeps.conv_cases()
    match = [c for c in groups if c.name == args.only_case]
    if not match:
        raise SystemExit(f"unknown case {args.only_case}; known: {[c.name for c in groups][:8]} ...")
    c = match[0]
    dist_kind = "uniform" if c.family in ("binary", "unary") else "normal"
    a = make_inputs(torch, c.dtype, c.in_elems[0], 1, dist_kind)
    b = make_inputs(torch, c.dtype, c.in_elems[1], 101, dist_kind) if len(c.in_elems) > 1 else None
    out = torch.empty(c.out_elems, dtype=torch_dtype(c.dtype), device="cuda")
    L = Launcher(lib_mod, c, {"a": a.data_ptr(), "b": b.data_ptr() if b is not None else None, "out": out.data_ptr()})
    ms = time_launches(torch, L.launch, max(1, args.steps), max(0, args.warmup))
    print(json.dumps({"case": c.name, "ms": round(ms, 4), "gbs": round(c.bytes / ms / 1e6, 1), "status": lib_mod.load().mx_last_error()}))


if __name__ == "__main__":
    main()
