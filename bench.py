#!/usr/bin/env python3
"""Benchmark of the sm_100a op library.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--exchange auto|multimem-exclusive|multimem|peer|copy|nccl]
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
# CPU arm: the oracle port of the reference's CPU backend on the host cores
# ---------------------------------------------------------------------------------------
def dispatch_overhead(torch, lib, iters=300):
    """Host-side cost of one op call made the reference's way (crates/maidenx_core/src/be/ops/binary.rs:112-163):
    cuda_malloc + cuda_memcpy_h2d of the metadata block, the op, cuda_free - on a 64-element add, so the kernel
    itself is negligible.  With the small-block pool the free no longer synchronises the device."""
    from maidenx_b200 import device
    a = torch.ones(64, device="cuda")
    b = torch.ones(64, device="cuda")
    o = torch.empty(64, device="cuda")
    meta = [64, 1, 1, 0, 0]
    out = {}
    for label, on in (("pooled_us_per_op", 1), ("cuda_malloc_free_us_per_op", 0)):
        lib.mx_set_small_pool(on)
        for _ in range(20):
            device.dispatch("add", "f32", meta, SZ(64), SZ(1), "META", a.data_ptr(), b.data_ptr(), o.data_ptr())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            device.dispatch("add", "f32", meta, SZ(64), SZ(1), "META", a.data_ptr(), b.data_ptr(), o.data_ptr())
        torch.cuda.synchronize()
        out[label] = round((time.perf_counter() - t0) / iters * 1e6, 2)
    lib.mx_set_small_pool(1)
    out["what"] = "cuda_malloc + cuda_memcpy_h2d(metadata) + cuda_add_f32(64 elements) + cuda_free through ctypes, host wall clock"
    return out


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
    """`--impl reference`: the reference's own CPU implementation of the path is a Rust crate that cannot be
    built here, so this arm times its CPU port (the oracle) on all host cores: the same model and step on a
    bounded sample of the batch.  Rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sample = 4
    steps = max(1, min(args.steps, 3))
    cb, best = cpu_mlp(sample, steps=steps + (1 if args.warmup > 0 else 0))
    line = {"metric": "mlp_train_samples_per_s", "value": cb["value"], "unit": "samples/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": min(args.warmup, 1), "ms_per_step": round(best * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 (element-type accumulation, as the reference's CPU backend)", "data": "synthetic", "impl": "reference",
            "config": {"workload": "MLP data-parallel training step: 4 x Linear(8192->8192) + GELU, MSE, SGD lr=1e-3",
                       "global_batch": MLP_GLOBAL_BATCH, "sample_rows": sample},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
# workload: data-parallel MLP training step (the headline at every N)
# ---------------------------------------------------------------------------------------
MLP_LAYERS, MLP_DIM, MLP_GLOBAL_BATCH, MLP_LR = 4, 8192, 16384, 1e-3
MLP_GEMMS_PER_STEP = 3 * MLP_LAYERS - 1       # dX of the first layer is not needed and not computed
# kernels launched per step: 11 GEMMs + 4 bias(/gelu) passes + 2 (mse, mse finish) + 3 gelu backward
# + 4 bias-gradient sums (partials folded inside the same launch) + 8 SGD updates (weights and bias per layer);
# with the NVLink exchange the 8 SGD launches become 4 x (barrier, fused reduce + update, barrier)
GEMM_DRAM_BYTES_PER_FLOP = 655.2e6 / 5.4976e11
MLP_KERNELS_PER_STEP = MLP_GEMMS_PER_STEP + MLP_LAYERS + 2 + (MLP_LAYERS - 1) + MLP_LAYERS + 2 * MLP_LAYERS


EXCHANGE_TEXT = {
    "none": "none (one rank)",
    "multimem": "own kernels over NVLink, fused with the SGD step: per layer a flag barrier, multimem.ld_reduce of this rank's 1/N shard of "
                "the bf16 gradients (in-switch f32 sum), f32 master update, multimem.st of the new bf16 weights to every rank; on a side "
                "stream beside the backward of the layers below",
    "peer": "own kernels over NVLink, fused with the SGD step: per layer a flag barrier, peer loads of this rank's 1/N shard of every rank's "
            "bf16 gradients, f32 master update, peer stores of the new bf16 weights to every rank; on a side stream beside the backward",
    "multimem-exclusive": "own kernel over NVLink, fused with the SGD step, on SMs of its own (the step's GEMMs run on the remaining SMs): per layer a "
                          "flag barrier, multimem.ld_reduce of this rank's 1/N shard of the bf16 gradients (in-switch f32 sum), f32 master update, "
                          "multimem.st of the new bf16 weights to every rank; on a side stream beside the backward of the layers below",
    "copy": "per layer, on a side stream beside the backward of the layers below: flag barrier, device-to-device copies (copy engines) of this "
            "rank's 1/N shard of every peer's bf16 gradients, one local kernel (f32 sum in rank order, f32 master update, new bf16 weights), "
            "copies of the new shard to every peer, flag barrier; no SM waits on NVLink",
    "nccl": "NCCL all-reduce, one bf16 bucket per layer, overlapped with backward; full-size SGD update on every rank",
}


def mlp_flops(batch):
    return MLP_GEMMS_PER_STEP * 2.0 * batch * MLP_DIM * MLP_DIM


def mlp_setup(torch, rank, world, dist=None, exchange="auto", exclusive_sms=8):
    from maidenx_b200.mlp import make_mlp
    local = MLP_GLOBAL_BATCH // world
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    x_all = torch.randn(MLP_GLOBAL_BATCH, MLP_DIM, device="cuda", generator=g).bfloat16()
    g.manual_seed(5)
    y_all = torch.randn(MLP_GLOBAL_BATCH, MLP_DIM, device="cuda", generator=g).bfloat16()
    x = x_all[rank * local:(rank + 1) * local].contiguous()
    y = y_all[rank * local:(rank + 1) * local].contiguous()
    del x_all, y_all
    torch.cuda.empty_cache()
    return make_mlp(MLP_LAYERS, MLP_DIM, local, "bf16", 6, torch, dist, world, exchange, exclusive_sms), x, y, local


def time_gemm(torch, lib_mod, local_batch, iters=10):
    """The dominant kernel alone: the forward product x . W^T of one layer, back to back."""
    M, N, K = local_batch, MLP_DIM, MLP_DIM
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).bfloat16()
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    meta = np.array([2, 2, 2, M, N, M, K, K, N, K, 1, 1, K, 0, 0], dtype=np.uint64)
    f = lib_mod.op("matmul", "bf16")
    ms = time_launches(torch, lambda: f(SZ(M * N), meta.ctypes.data, x.data_ptr(), w.data_ptr(), c.data_ptr()), iters, 3)
    return ms, 2.0 * M * N * K


def e2e_mlp(torch, lib, mlp, x, y, dist, world, steps, warm):
    """The same step fed from pinned host memory: every step copies its shard's inputs host -> device and reads the
    loss back.  The copies of step i + 1 run on a copy stream into the second of two device buffers while step i
    computes (an input pipeline: the user-facing loop of maidenx_b200.mlp.InputPipeline)."""
    from maidenx_b200.mlp import InputPipeline
    hx, hy = x.cpu().pin_memory(), y.cpu().pin_memory()
    nbytes = x.numel() * x.element_size()
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    pipe = InputPipeline(torch, x, y)

    def run(n):
        pipe.prefetch(hx, hy)
        for i in range(n):
            xb, yb = pipe.next_batch()          # the compute stream now waits for this batch's copies
            if i + 1 < n:
                pipe.prefetch(hx, hy)           # next batch: copies overlap this step
            mlp.train_step(xb.data_ptr(), yb.data_ptr(), MLP_LR, torch, dist, world)
            pipe.release()                      # the buffers may be overwritten once this step's kernels are done
            lib.cuda_memcpy_d2h(loss_host.data_ptr(), mlp.ptr("loss_ptr"), 4)

    run(warm)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    run(steps)
    torch.cuda.synchronize()
    dt_s = (time.perf_counter() - t0) / steps
    if world > 1:
        t = torch.tensor([dt_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt_s = float(t.item())
    return {"value": round(MLP_GLOBAL_BATCH / dt_s, 1), "unit": "samples/s", "h2d_bytes_per_step": 2 * nbytes * world, "d2h_bytes_per_step": 4 * world,
            "steps": steps, "ms_per_step": round(dt_s * 1e3, 3), "loss": float(loss_host[0]),
            "pipeline": "double-buffered: host->device copies of step i+1 on a copy stream while step i computes"}


def cpu_mlp(sample_batch, steps=1):
    """The CPU arm: the same model and step composed from the CPU port of the reference's backend, on a
    bounded sample of the batch (full 4 x 8192^2 weights, `sample_batch` rows)."""
    from oracle import binding, mlp_reference
    from maidenx_b200 import dtypes as D
    binding.load()
    binding.set_num_threads(os.cpu_count() or 1)  # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1)
    binding.set_reduce_parallel(True)
    rng = np.random.default_rng(6)
    bound = 1.0 / np.sqrt(MLP_DIM)
    W = [D.encode(rng.uniform(-bound, bound, MLP_DIM * MLP_DIM).astype(np.float32), D.BF16) for _ in range(MLP_LAYERS)]
    b = [D.encode(rng.uniform(-bound, bound, 1).astype(np.float32), D.BF16) for _ in range(MLP_LAYERS)]
    x = D.encode(rng.standard_normal(sample_batch * MLP_DIM).astype(np.float32), D.BF16)
    y = D.encode(rng.standard_normal(sample_batch * MLP_DIM).astype(np.float32), D.BF16)
    m = mlp_reference.CpuMlp(MLP_LAYERS, MLP_DIM, sample_batch, "bf16", W, b)
    best = None
    for _ in range(steps):
        t0 = time.perf_counter()
        m.step(x, y, MLP_LR)
        dt_s = time.perf_counter() - t0
        best = dt_s if best is None else min(best, dt_s)
    return {"value": round(sample_batch / best, 3), "unit": "samples/s", "cores": binding.max_threads(), "kind": "port",
            "sample": f"one full training step (4 x Linear(8192->8192), GELU, MSE, SGD, bf16) on {sample_batch} of the 16384 rows, "
                      f"{best:.1f} s; weights and update at full size"}, best


# ---------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweeps", action="store_true", help="skip the per-case tables (reductions, conv)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--global-batch", type=int, default=None,
                    help="tuning aid: another global batch than the benchmark's 16384 (the JSON line says so; not a headline number)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "multimem-exclusive", "copy", "multimem", "peer", "nccl"],
                    help="N > 1: how gradients are exchanged (auto: the library's NVLink kernels, NCCL if symmetric memory is unavailable)")
    ap.add_argument("--exchange-sms", type=int, default=8, help="multimem-exclusive: SMs given to the exchange kernel")
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
    if args.global_batch:
        global MLP_GLOBAL_BATCH
        MLP_GLOBAL_BATCH = args.global_batch
    if MLP_GLOBAL_BATCH % world != 0:
        raise SystemExit("the global batch must divide evenly over the ranks")
    mlp, x, y, local_batch = mlp_setup(torch, rank, world, dist if world > 1 else None, args.exchange, args.exchange_sms)

    def step():
        mlp.train_step(x.data_ptr(), y.data_ptr(), MLP_LR, torch, dist, world)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(args.steps):
        step()
    if hasattr(mlp, "join"):
        mlp.join()  # the exchange of the last step runs on a side stream: the closing event waits for it
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_step = s.elapsed_time(e) / args.steps
    if world > 1:
        t = torch.tensor([ms_step], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())
    loss = mlp.loss()
    mlp_exchange = mlp.exchange
    if hasattr(mlp, "status") and mlp.status() != 0:
        raise RuntimeError(f"a cross-rank barrier gave up waiting for rank {mlp.status() - 1}")
    lib.mx_device_synchronize()
    if lib.mx_last_error():
        raise RuntimeError(f"op library reported status {lib.mx_last_error()} at {lib.mx_last_error_where().decode()}")
    value = MLP_GLOBAL_BATCH / (ms_step / 1e3)

    # the dominant kernel alone, live, on this rank's shapes
    gemm_ms, gemm_flops = time_gemm(torch, lib_mod, local_batch)
    e2e = None if args.no_e2e else e2e_mlp(torch, lib, mlp, x, y, dist, world, steps=6, warm=2)
    clocks = sampler.stop()

    sweeps_out, roofline, cpu = {}, None, None
    if rank == 0:
        achieved = gemm_flops / gemm_ms / 1e9
        # DRAM bytes per launch: the ncu capture of this kernel at [8192, 4096] x 8192 read 595.1 MB and
        # wrote 60.1 MB for 5.4976e11 flop; same K, tile shape and tile order here, so traffic scales
        # with the number of output tiles, i.e. with the flops
        traffic = int(GEMM_DRAM_BYTES_PER_FLOP * gemm_flops)
        roofline = {"bound": "tensor", "kernel": "tc_gemm_kernel", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": round(achieved / peaks["bf16_tflops"], 4), "peak_source": peaks["source"] + " (burst: kernel timed alone)",
                    "launch_shape": f"[{local_batch},{MLP_DIM}] x [{MLP_DIM},{MLP_DIM}]^T bf16", "flops_per_launch": gemm_flops,
                    "ms_per_launch": round(gemm_ms, 4), "traffic": traffic,
                    "step_gemm_share": round(MLP_GEMMS_PER_STEP * gemm_ms / ms_step, 3),
                    "step_tflops": round(mlp_flops(local_batch) * world / ms_step / 1e9, 1),
                    "step_frac_of_sustained": round(mlp_flops(local_batch) / ms_step / 1e9 / peaks["bf16_tflops_sustained"], 4)}
    del mlp, x, y
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_sweeps:
        groups = (("elementwise", sweeps.elementwise_cases(), (1, 101), "uniform"), ("reduction", sweeps.reduction_cases(), (3, 103), "normal"),
                  ("conv", sweeps.conv_cases(), (10, 110), "normal"))
        for name, cases, seeds, kind in groups:
            rows = run_sweep_group(torch, lib_mod, cases, 10, 3, seeds, kind)
            for r in rows:
                r["frac"] = round(r["gbs"] / peaks["hbm_gbs"], 4)
            sweeps_out[name] = rows
        ew = sweeps_out["elementwise"]
        sweeps_out["summary"] = {
            "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"], "nominal_gbs": NOMINAL_HBM_GBS,
            "elementwise_aggregate_gbs": round(sum(r["bytes"] for r in ew) / sum(r["ms"] for r in ew) / 1e6, 1),
            "cases_at_or_above_80pct_of_measured": sum(1 for g in ("elementwise", "reduction", "conv") for r in sweeps_out[g] if r["frac"] >= 0.8),
            "cases": sum(len(sweeps_out[g]) for g in ("elementwise", "reduction", "conv"))}
        sweeps_out["dispatch"] = dispatch_overhead(torch, lib)
        if lib.mx_last_error():
            raise RuntimeError(f"op library reported status {lib.mx_last_error()} at {lib.mx_last_error_where().decode()}")
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = cpu_mlp(4)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        line = {"metric": "mlp_train_samples_per_s", "value": round(value, 1), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16 (f32 accumulate, f32 master weights)",
                "data": "synthetic (seeded N(0,1) inputs and targets, Kaiming-uniform weights U(-1/sqrt(8192), 1/sqrt(8192)))",
                "config": {"workload": "MLP data-parallel training step: 4 x Linear(8192->8192) + GELU, MSE, SGD lr=1e-3", "global_batch": MLP_GLOBAL_BATCH,
                           "per_gpu_batch": local_batch, "parallelism": f"dp{world}", "allreduce": EXCHANGE_TEXT[mlp_exchange],
                           "l2": "per-step working set (weights 0.5 GB + activations 2 GB per GPU at N=1) far exceeds the 126 MB L2"},
                "loss": loss, "clocks": clocks, "gpu_launches": (MLP_KERNELS_PER_STEP + (3 * MLP_LAYERS - 2 * MLP_LAYERS if mlp_exchange in ("multimem", "multimem-exclusive", "peer", "copy") else 0)) * args.steps, "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu,
                "sweeps": sweeps_out}
        print(json.dumps(line))


def run_only_case(torch, lib_mod, args):
    """Launch one sweep case a few times (for ncu captures of a single kernel)."""
    if args.small:
        groups = sweeps.elementwise_cases(8192, 8192) + sweeps.reduction_cases(4096, 16384, (16, 512, 4096)) + sweeps.conv_cases(N=16)
    else:
        groups = sweeps.elementwise_cases() + sweeps.reduction_cases() + sweeps.conv_cases()
    if args.only_case.startswith("gemm_"):
        # gemm_<bf16|f16|f32>[_<MxNxK>]: the forward product x . W^T of one MLP layer; --small: 8192 x 4096 x 8192 (above L2)
        parts = args.only_case.split("_")
        dt = parts[1]
        M, N, K = (8192, 4096, 8192) if args.small else (MLP_GLOBAL_BATCH, MLP_DIM, MLP_DIM)
        if len(parts) > 2:
            M, N, K = (int(v) for v in parts[2].split("x"))
        x = torch.randn(M, K, device="cuda").to(torch_dtype(dt))
        w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch_dtype(dt))
        c = torch.empty(M, N, device="cuda", dtype=torch_dtype(dt))
        meta = np.array([2, 2, 2, M, N, M, K, K, N, K, 1, 1, K, 0, 0], dtype=np.uint64)
        f = lib_mod.op("matmul", dt)
        ms = time_launches(torch, lambda: f(SZ(M * N), meta.ctypes.data, x.data_ptr(), w.data_ptr(), c.data_ptr()), max(1, args.steps), max(0, args.warmup))
        lib_mod.load().mx_device_synchronize()
        print(json.dumps({"case": args.only_case, "shape": [M, N, K], "ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1),
                          "status": lib_mod.load().mx_last_error()}))
        return
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
