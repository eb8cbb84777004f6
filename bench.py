#!/usr/bin/env python3
"""Benchmark of the sm_100a op library.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--exchange auto|multimem-exclusive|multimem|peer|copy|nccl]
    python bench.py --impl reference ...      # the CPU arm: the oracle port on the host cores

One JSON line is printed by rank 0.  `value` is whole-job throughput of the MLP training step with inputs
resident in HBM; `e2e` is the same metric with host buffers (copies inside the timed region); `roofline`
describes the dominant kernel (timed in bursts, with the SM clock seen during each burst) and carries the compact
summary of every single-op sweep; `cpu_baseline` is the CPU port of the reference's backend timed on this box;
`sweeps` lists every single-op case with its achieved HBM GB/s (or TFLOP/s), the CPU port's figure on a bounded
sample beside it, and whether a sample of the full-size output was checked against the CPU oracle.
torch is used for device memory, events and (N > 1) torch.distributed; every op in the timed regions is a call
into libmaidenx_cuda.so.  The oracle is imported only by the CPU legs and by the output checks.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
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
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_HBM_GBS = 6650.0         # used only when MEASURED_PEAKS.json is absent
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def profiled_traffic(kernel, shape_key):
    """DRAM bytes per launch and the work it was captured on, from the committed ncu table
    (profiles/dram_traffic_per_launch.md: | kernel | shape | dram_read_bytes | dram_write_bytes | work | unit |)."""
    p = ROOT / "profiles" / "dram_traffic_per_launch.md"
    if not p.exists():
        return None
    for line in p.read_text().splitlines():
        f = [x.strip().strip("`") for x in line.strip().strip("|").split("|")]
        if len(f) >= 6 and f[0] == kernel and f[1] == shape_key:
            try:
                return {"read": float(f[2]), "write": float(f[3]), "work": float(f[4]), "unit": f[5]}
            except ValueError:
                return None
    return None


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



class ClockProbe:
    """SM clock right now, through NVML (read-only query); used to tag each timing burst with the clock the GPU ran at."""

    def __init__(self, device_index):
        self.h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        except Exception:
            self.h = None

    def sm_mhz(self):
        if self.h is None:
            return None
        try:
            return int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
        except Exception:
            return None


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
        elif c.family == "fold":
            self.args = (SZ(c.num_els), SZ(3), m, bufs["a"], bufs["out"])
        elif c.family == "softmax":
            self.args = (SZ(c.num_els), SZ(2), SZ(c.extra["dim"]), m, bufs["a"], bufs["out"])
        elif c.family in ("pad", "pad_backward"):
            self.args = (SZ(c.num_els), SZ(c.extra["n_out"]), SZ(4), m, bufs["a"], bufs["out"]) + pad_value_arg(c)
        else:
            raise KeyError(c.family)

    def launch(self):
        self.fn(*self.args)


def pad_value_arg(c):
    """The by-value fill constant of pad_with_constant (0.5); the other padding entry points take none."""
    if not c.extra.get("constant"):
        return ()
    from maidenx_b200 import dtypes as D
    return (D.scalar_arg(0.5, D.BY_NAME[c.dtype]),)


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



# ---------------------------------------------------------------------------------------
# output checks: a sample of each full-size result against the CPU oracle (the checker, never the thing timed)
# ---------------------------------------------------------------------------------------
NP_STORE = {"f32": np.float32, "bf16": np.uint16, "f16": np.float16, "i32": np.int32, "f64": np.float64}
EXACT_OPS = {"add", "sub", "mul", "div", "neg", "relu", "max", "min"}


def to_store(t):
    """torch tensor -> numpy array of stored bits (bf16 as uint16)."""
    import torch
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1)
    return t.cpu().numpy().reshape(-1)


def decode(arr, dt):
    from maidenx_b200 import dtypes as D
    return D.decode(arr, D.BY_NAME[dt]).astype(np.float64) if dt != "i32" else arr.astype(np.float64)


def close(got, ref, dt, rel, scale):
    """|got - ref| <= rel * max(|ref|, scale), NaN and infinity patterns equal; rel == 0: same bits (NaNs as a class)."""
    if dt == "i32":
        return bool(np.array_equal(got, ref))
    g, r = decode(got, dt), decode(ref, dt)
    if not np.array_equal(np.isnan(g), np.isnan(r)):
        return False
    ok = ~np.isnan(r)
    g, r = g[ok], r[ok]
    sc = np.broadcast_to(np.asarray(scale, dtype=np.float64), ok.shape)[ok] if np.ndim(scale) else np.full(r.shape, float(scale))
    inf = np.isinf(r)
    if not np.array_equal(g[inf], r[inf]) or np.isinf(g[~inf]).any():
        return False
    g, r, sc = g[~inf], r[~inf], sc[~inf]
    if rel == 0.0:
        return bool(np.array_equal(g, r))
    return bool(np.all(np.abs(g - r) <= rel * np.maximum(np.abs(r), np.maximum(sc, 1e-30))))


def oracle_call(op, dt, *args):
    from oracle import binding
    binding.op(op, dt)(*args)


def sample_rows(n, count, seed):
    rows = {0, 1, n // 2, n - 2, n - 1, 63, 64, 65}
    rng = np.random.default_rng(seed)
    while len(rows) < count:
        rows.add(int(rng.integers(0, n)))
    return np.array(sorted(r for r in rows if 0 <= r < n))[:count]


def verify_case(torch, c, a, b, out):
    """Compares a sample of `out` (the result of the last timed launch of sweep case `c`) with the oracle run on just
    that sample.  Elementwise: whole output rows (every 64-wide column tile of the transposed layouts is crossed);
    reductions: whole output elements (all their terms); im2col / col2im: whole images."""
    from oracle import binding
    dt = c.dtype
    st = NP_STORE[dt]
    tdt = torch_dtype(dt)
    if c.family in ("binary", "unary"):
        R, C = c.metadata[0], c.metadata[1]
        rows = sample_rows(R, 12, C)
        idx = torch.as_tensor(rows, device="cuda")

        def logical(buf, strides, off):
            v = torch.as_strided(buf, (R, C), tuple(int(s) for s in strides), int(off))
            return to_store(v[idx])

        n = len(rows) * C
        got = to_store(out[:R * C].view(R, C)[idx])
        ref = np.empty(n, st)
        meta = np.asarray([n, 1, 1, 0, 0] if c.family == "binary" else [n, 1, 0], dtype=np.uint64)
        la = logical(a, c.metadata[2:4], c.metadata[6] if c.family == "binary" else c.metadata[4])
        if c.family == "binary":
            lb = logical(b, c.metadata[4:6], c.metadata[7])
            oracle_call(c.op, dt, SZ(n), SZ(1), meta.ctypes.data, la.ctypes.data, lb.ctypes.data, ref.ctypes.data)
        else:
            oracle_call(c.op, dt, SZ(n), SZ(1), meta.ctypes.data, la.ctypes.data, ref.ctypes.data)
        if c.op in EXACT_OPS:
            return close(got, ref, dt, 0.0, 0.0)
        rel = 1e-5 if dt == "f32" else 1e-2
        return close(got, ref, dt, rel, np.abs(decode(la, dt)) if c.op == "gelu" else 0.0)
    if c.family == "reduce":
        R, C = c.metadata[0], c.metadata[1]
        dim0 = c.metadata[5] == C  # stride of the reduced dim: C for dim 0, 1 for dim 1
        x = a[:R * C].view(R, C)
        binding.set_wide(True)
        try:
            if dim0:
                cols = sample_rows(C, 64, R)
                sub = to_store(x[:, torch.as_tensor(cols, device="cuda")])
                m = np.asarray([R, 64, 64, 1, R, 64, 0], dtype=np.uint64)
                ref = np.empty(64, st)
                oracle_call(c.op, dt, SZ(R * 64), SZ(2), SZ(1), m.ctypes.data, sub.ctypes.data, ref.ctypes.data)
                got = to_store(out[:C][torch.as_tensor(cols, device="cuda")])
                terms = R
            else:
                rows = sample_rows(R, 64, C)
                sub = to_store(x[torch.as_tensor(rows, device="cuda")])
                m = np.asarray([64, C, C, 1, C, 1, 0], dtype=np.uint64)
                ref = np.empty(64, st)
                oracle_call(c.op, dt, SZ(64 * C), SZ(2), SZ(1), m.ctypes.data, sub.ctypes.data, ref.ctypes.data)
                got = to_store(out[:R][torch.as_tensor(rows, device="cuda")])
                terms = C
        finally:
            binding.set_wide(False)
        if c.op == "max" or dt == "i32":
            return close(got, ref, dt, 0.0, 0.0)
        scale = np.sqrt(terms) / (terms if c.op == "mean" else 1)
        return close(got, ref, dt, 1e-4 if dt == "f32" else 2e-2, scale)
    if c.family == "sum_to_shape":
        A, B, Cc = c.metadata[0:3]
        cols = sample_rows(Cc, 32, A)
        sub = to_store(a[:A * B * Cc].view(A, B, Cc)[:, :, torch.as_tensor(cols, device="cuda")])
        m = np.asarray([A, B, 32, B * 32, 32, 1, 1, 1, 32, 0], dtype=np.uint64)
        ref = np.empty(32, st)
        binding.set_wide(True)
        try:
            oracle_call("sum_to_shape", dt, SZ(A * B * 32), SZ(3), m.ctypes.data, sub.ctypes.data, ref.ctypes.data)
        finally:
            binding.set_wide(False)
        got = to_store(out[:Cc][torch.as_tensor(cols, device="cuda")])
        return close(got, ref, dt, 1e-4 if dt == "f32" else 2e-2, np.sqrt(A * B))
    if c.family in ("im2col", "col2im"):
        Bn, Cin, H, W, kh, kw, oh, ow = c.metadata[:8]
        x_img, col_img = Cin * H * W, Cin * kh * kw * oh * ow
        m = np.asarray([1] + list(c.metadata[1:]), dtype=np.uint64)
        ok = True
        for img in (0, Bn - 1):
            if c.family == "im2col":
                src = to_store(a[img * x_img:(img + 1) * x_img])
                ref = np.empty(col_img, st)
                oracle_call(c.op, dt, SZ(col_img), m.ctypes.data, src.ctypes.data, ref.ctypes.data)
                got = to_store(out[img * col_img:(img + 1) * col_img])
            else:
                src = to_store(a[img * col_img:(img + 1) * col_img])
                ref = np.empty(x_img, st)
                oracle_call(c.op, dt, SZ(col_img), m.ctypes.data, src.ctypes.data, ref.ctypes.data)
                got = to_store(out[img * x_img:(img + 1) * x_img])
            ok = ok and close(got, ref, dt, 0.0, 0.0)
        return ok
    if c.family == "fold":
        # whole rows of the [rows, windows, size] gradient
        R, Wn, Sz = c.extra["rows"], c.extra["windows"], c.extra["size"]
        F = Wn - 1 + Sz
        idx = torch.as_tensor(sample_rows(R, 12, Wn), device="cuda")
        sub = to_store(a[:R * Wn * Sz].view(R, Wn * Sz)[idx])
        got = to_store(out[:R * F].view(R, F)[idx])
        k = len(idx)
        m = np.asarray([k, Wn, Sz, Wn * Sz, Sz, 1, 1, 2, F, 1, Sz, 0], dtype=np.uint64)
        ref = np.empty(k * F, st)
        binding.set_wide(True)
        try:
            oracle_call("fold", dt, SZ(k * Wn * Sz), SZ(3), m.ctypes.data, sub.ctypes.data, ref.ctypes.data)
        finally:
            binding.set_wide(False)
        return close(got, ref, dt, 1e-5 if dt == "f32" else 1e-2, 2.0)
    if c.family == "softmax":
        R, C = c.metadata[0], c.metadata[1]
        x, y = a[:R * C].view(R, C), out[:R * C].view(R, C)
        if c.extra["dim"] == 1:   # whole rows
            idx = torch.as_tensor(sample_rows(R, 12, C), device="cuda")
            sub, got, shape = to_store(x[idx]), to_store(y[idx]), (len(idx), C)
        else:                     # whole columns
            idx = torch.as_tensor(sample_rows(C, 64, R), device="cuda")
            sub, got, shape = to_store(x[:, idx]), to_store(y[:, idx]), (R, len(idx))
        m = np.asarray([shape[0], shape[1], shape[1], 1, 0], dtype=np.uint64)
        ref = np.empty(shape[0] * shape[1], st)
        binding.set_wide(True)   # exp and the sum in f32 for 16-bit inputs, as the kernel computes them
        try:
            oracle_call("softmax", dt, SZ(ref.size), SZ(2), SZ(c.extra["dim"]), m.ctypes.data, sub.ctypes.data, ref.ctypes.data)
        finally:
            binding.set_wide(False)
        return close(got, ref, dt, 1e-5 if dt == "f32" else 2e-2, 1e-30 if dt == "f32" else 1e-4)
    if c.family in ("pad", "pad_backward"):
        # whole images: the first and the last of the batch
        Bn, Cc, H, W = c.metadata[0:4]
        Ho, Wo = c.metadata[11], c.metadata[12]
        in_img, out_img = Cc * H * W, Cc * Ho * Wo
        m = np.asarray([1] + list(c.metadata[1:9]) + [1] + list(c.metadata[10:]), dtype=np.uint64)
        ok = True
        for img in (0, Bn - 1):
            if c.family == "pad":
                src = to_store(a[img * in_img:(img + 1) * in_img])
                ref = np.empty(out_img, st)
                oracle_call(c.op, dt, SZ(in_img), SZ(out_img), SZ(4), m.ctypes.data, src.ctypes.data, ref.ctypes.data, *pad_value_arg(c))
                got = to_store(out[img * out_img:(img + 1) * out_img])
            else:
                src = to_store(a[img * out_img:(img + 1) * out_img])
                ref = np.empty(in_img, st)
                oracle_call(c.op, dt, SZ(in_img), SZ(out_img), SZ(4), m.ctypes.data, src.ctypes.data, ref.ctypes.data)
                got = to_store(out[img * in_img:(img + 1) * in_img])
            ok = ok and close(got, ref, dt, 0.0, 0.0)
        return ok
    raise KeyError(c.family)


def verify_gemm(torch, dt, M, N, K, a, b, c, a_major="k", b_major="k", rows=16):
    """Sampled rows of C = A . B against the wide-accumulating oracle (its matmul is row-independent)."""
    from oracle import binding
    st = NP_STORE[dt]
    r = sample_rows(M, rows, N)
    idx = torch.as_tensor(r, device="cuda")
    a_rows = to_store(a.view(M, K)[idx] if a_major == "k" else a.view(K, M)[:, idx].t())
    bs = to_store(b)
    bst = [1, K] if b_major == "k" else [N, 1]
    meta = np.asarray([2, 2, 2, len(r), N, len(r), K, K, N, K, 1] + bst + [0, 0], dtype=np.uint64)
    ref = np.empty(len(r) * N, st)
    binding.set_wide(True)
    try:
        oracle_call("matmul", dt, SZ(len(r) * N), meta.ctypes.data, a_rows.ctypes.data, bs.ctypes.data, ref.ctypes.data)
    finally:
        binding.set_wide(False)
    got = to_store(c.view(M, N)[idx])
    return close(got, ref, dt, 1e-4 if dt == "f32" else 2e-2, np.sqrt(K))


# ---------------------------------------------------------------------------------------
# CPU figures: the oracle (the CPU port of the reference's backend) on a bounded sample of each case
# ---------------------------------------------------------------------------------------
def cpu_inputs(rng, dt, n, dist):
    from maidenx_b200 import dtypes as D
    if dt == "i32":
        return rng.integers(-1000, 1001, n).astype(np.int32)
    v = rng.uniform(-1, 1, n) if dist == "uniform" else rng.standard_normal(n)
    return D.encode(v.astype(np.float32), D.BY_NAME[dt])


def cpu_time_cases(cases, dist, passes=2):
    """Seconds per call of each case on the oracle, all host threads, best of `passes`."""
    from oracle import binding
    binding.load()
    binding.set_num_threads(os.cpu_count() or 1)
    binding.set_reduce_parallel(True)
    rng = np.random.default_rng(1)
    pools = {}
    out = []
    for c in cases:
        key = c.dtype
        na = max(c.in_elems[0], 1)
        nb = c.in_elems[1] if len(c.in_elems) > 1 else 0
        if key not in pools or pools[key][0].size < na or pools[key][1].size < max(nb, 1) or pools[key][2].size < c.out_elems:
            pools[key] = (cpu_inputs(rng, c.dtype, na, dist), cpu_inputs(rng, c.dtype, max(nb, 1), dist), np.empty(max(c.out_elems, 1), NP_STORE[c.dtype]))
        a, b, o = pools[key]
        m = np.asarray(c.metadata, dtype=np.uint64)
        if c.family == "binary":
            args = (SZ(c.num_els), SZ(2), m.ctypes.data, a.ctypes.data, b.ctypes.data, o.ctypes.data)
        elif c.family == "unary":
            args = (SZ(c.num_els), SZ(2), m.ctypes.data, a.ctypes.data, o.ctypes.data)
        elif c.family == "reduce":
            args = (SZ(c.num_els), SZ(2), SZ(c.extra["num_red"]), m.ctypes.data, a.ctypes.data, o.ctypes.data)
        elif c.family == "sum_to_shape":
            args = (SZ(c.num_els), SZ(3), m.ctypes.data, a.ctypes.data, o.ctypes.data)
        elif c.family == "fold":
            args = (SZ(c.num_els), SZ(3), m.ctypes.data, a.ctypes.data, o.ctypes.data)
        elif c.family == "softmax":
            args = (SZ(c.num_els), SZ(2), SZ(c.extra["dim"]), m.ctypes.data, a.ctypes.data, o.ctypes.data)
        elif c.family in ("pad", "pad_backward"):
            args = (SZ(c.num_els), SZ(c.extra["n_out"]), SZ(4), m.ctypes.data, a.ctypes.data, o.ctypes.data) + pad_value_arg(c)
        else:
            args = (SZ(c.num_els), m.ctypes.data, a.ctypes.data, o.ctypes.data)
        fn = binding.op(c.op, c.dtype)
        best = None
        for _ in range(passes):
            t0 = time.perf_counter()
            fn(*args)
            dt_s = time.perf_counter() - t0
            best = dt_s if best is None else min(best, dt_s)
        out.append(best)
    return out, binding.max_threads()


def run_sweep_group(torch, lib_mod, cases, small_cases, iters, warm, seeds, dist, peaks, verify, with_cpu):
    """Per-case device timing (CUDA events, inputs larger than L2), the oracle's GB/s on the reduced-size twin of the
    case, and the output check.  Inputs are allocated per dtype once."""
    rows = []
    cpu_s, cores = cpu_time_cases(small_cases, dist) if with_cpu else ([None] * len(cases), None)
    cpu_of = {c.name.split("/")[0] + "/" + str(i): (s, sc) for i, (c, s, sc) in enumerate(zip(cases, cpu_s, small_cases))}
    by_dtype = {}
    for i, c in enumerate(cases):
        by_dtype.setdefault(c.dtype, []).append((i, c))
    for dt, cs in by_dtype.items():
        na = max(c.in_elems[0] for _, c in cs)
        nb = max((c.in_elems[1] for _, c in cs if len(c.in_elems) > 1), default=0)
        no = max(c.out_elems for _, c in cs)
        a = make_inputs(torch, dt, na, seeds[0], dist)
        b = make_inputs(torch, dt, nb, seeds[1], dist) if nb else None
        if dt != "i32" and b is not None:
            b = torch.where(b == 0, torch.ones_like(b), b)  # keep div on its arithmetic path
        out = torch.empty(no, dtype=torch_dtype(dt), device="cuda")
        bufs = {"a": a.data_ptr(), "b": b.data_ptr() if b is not None else None, "out": out.data_ptr()}
        for i, c in cs:
            L = Launcher(lib_mod, c, bufs)
            ms = time_launches(torch, L.launch, iters, warm)
            row = {"case": c.name, "ms": round(ms, 4), "gbs": round(c.bytes / ms / 1e6, 1), "bytes": c.bytes,
                   "frac": round(c.bytes / ms / 1e6 / peaks["hbm_gbs"], 4)}
            s, sc = cpu_of[c.name.split("/")[0] + "/" + str(i)]
            if s is not None:
                row["cpu_gbs"] = round(sc.bytes / s / 1e9, 3)
                row["cpu_sample_elems"] = sc.num_els
            if verify:
                row["verified"] = bool(verify_case(torch, c, a, b, out))
            rows.append((i, row))
        del a, b, out
        torch.cuda.empty_cache()
    rows = [r for _, r in sorted(rows, key=lambda t: t[0])]
    return rows, cores

# ---------------------------------------------------------------------------------------
# products: the tensor-core kernels and the SIMT kernel, stand-alone
# ---------------------------------------------------------------------------------------
def gemm_operands(torch, dt, M, N, K, a_major="k", b_major="k", seed=21):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    tdt = torch_dtype(dt)
    a = torch.randn((M, K) if a_major == "k" else (K, M), device="cuda", generator=g).to(tdt)
    b = (torch.randn((N, K) if b_major == "k" else (K, N), device="cuda", generator=g) / K ** 0.5).to(tdt)
    c = torch.empty(M, N, device="cuda", dtype=tdt)
    ast = [K, 1] if a_major == "k" else [1, M]
    bst = [1, K] if b_major == "k" else [N, 1]
    meta = np.array([2, 2, 2, M, N, M, K, K, N] + ast + bst + [0, 0], dtype=np.uint64)
    return a, b, c, meta


def gemm_row(torch, lib_mod, name, dt, M, N, K, a_major, b_major, peak_tflops, iters, verify, kernel):
    a, b, c, meta = gemm_operands(torch, dt, M, N, K, a_major, b_major)
    f = lib_mod.op("matmul", dt)
    ms = time_launches(torch, lambda: f(SZ(M * N), meta.ctypes.data, a.data_ptr(), b.data_ptr(), c.data_ptr()), iters, 3)
    tf = 2.0 * M * N * K / ms / 1e9
    row = {"case": name, "kernel": kernel, "shape": [M, N, K], "ms": round(ms, 4), "tflops": round(tf, 1),
           "frac_of_bf16_peak": round(tf / peak_tflops, 4)}
    if verify:
        row["verified"] = bool(verify_gemm(torch, dt, M, N, K, a, b, c, a_major, b_major))
    return row


def time_gemm_bursts(torch, lib_mod, probe, M, N, K, bursts=6, per_burst=12):
    """The dominant kernel alone: the forward product x . W^T of one layer, in `bursts` bursts of `per_burst`
    back-to-back launches (CUDA events around each burst); the SM clock is read through NVML while each burst runs."""
    a, b, c, meta = gemm_operands(torch, "bf16", M, N, K)
    f = lib_mod.op("matmul", "bf16")

    def launch():
        f(SZ(M * N), meta.ctypes.data, a.data_ptr(), b.data_ptr(), c.data_ptr())

    for _ in range(5):
        launch()
    torch.cuda.synchronize()
    out = []
    for _ in range(bursts):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(per_burst):
            launch()
        e.record()
        mhz = []
        while not e.query():
            v = probe.sm_mhz()
            if v:
                mhz.append(v)
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / per_burst
        out.append({"ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1), "sm_mhz": int(np.median(mhz)) if mhz else None})
    return out, (a, b, c)


def gemm_same_method_as_peak(torch, lib_mod, M, N, K, bufs):
    """The peak this kernel is held against was measured as the best of 10 single launches of the library's GEMM and as
    a seconds-long loop.  The same two methods on this box, at this moment, for the library's GEMM (torch.matmul, the
    comparison point - never the product path) and for tc_gemm_kernel, on the same operands: best of 10 single launches
    (a synchronisation between them) and one burst of 12, library first."""
    a, b, c = bufs
    meta = np.array([2, 2, 2, M, N, M, K, K, N, K, 1, 1, K, 0, 0], dtype=np.uint64)
    f = lib_mod.op("matmul", "bf16")
    c2 = torch.empty_like(c)
    runs = {"library_gemm": lambda: torch.matmul(a, b.t(), out=c2),
            "tc_gemm_kernel": lambda: f(SZ(M * N), meta.ctypes.data, a.data_ptr(), b.data_ptr(), c.data_ptr())}
    flops = 2.0 * M * N * K
    out = {}
    for name, fn in runs.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e)
            best = ms if best is None else min(best, ms)
        burst = time_launches(torch, fn, 12, 0)
        out[name] = {"best_of_10_tflops": round(flops / best / 1e9, 1), "burst_of_12_tflops": round(flops / burst / 1e9, 1)}
    return out


# ---------------------------------------------------------------------------------------
# Conv2d as a whole (BASELINE config 5): the layer composed from the library's ops
# ---------------------------------------------------------------------------------------
CONV = dict(B=64, C=256, H=56, W=56, Co=256, k=3, s=1, p=1)


def conv_rows(torch, lib_mod, peaks, iters, verify, small=False):
    """Forward and backward of the Conv2d layer in bf16 and f32, in the literal reference call sequence (mode 0) and
    the direct form (mode 1), plus the three products of the literal form alone.  FLOP = 2 * B*P * K * Cout per product."""
    from maidenx_b200 import _lib
    lib = lib_mod.load()
    cv = dict(CONV)
    if small:
        cv["B"] = 8
    B, C, H, W, Co, k = cv["B"], cv["C"], cv["H"], cv["W"], cv["Co"], cv["k"]
    P, K = H * W, C * k * k
    conv = _lib.MxConv2d(B, C, H, W, Co, k, k, cv["s"], cv["s"], cv["p"], cv["p"])
    flop = 2.0 * B * P * K * Co
    rows = []
    for dt in ("bf16", "f32"):
        tdt = torch_dtype(dt)
        g = torch.Generator(device="cuda")
        g.manual_seed(10)
        x = torch.randn(B * C * H * W, device="cuda", generator=g).to(tdt)
        g.manual_seed(11)
        bound = 1.0 / K ** 0.5
        w = ((torch.rand(Co * K, device="cuda", generator=g) * 2 - 1) * bound).to(tdt)
        bias = ((torch.rand(Co, device="cuda", generator=g) * 2 - 1) * bound).to(tdt)
        go = torch.randn(B * Co * P, device="cuda", generator=g).to(tdt)
        cols = torch.empty(lib.mx_conv2d_cols_elems(ctypes.byref(conv)), device="cuda", dtype=tdt)
        ws = torch.empty(max(lib.mx_conv2d_workspace_elems(ctypes.byref(conv), m, bw) for m in (0, 1) for bw in (0, 1)), device="cuda", dtype=tdt)
        out = torch.empty(B * Co * P, device="cuda", dtype=tdt)
        gx, gw, gb = torch.empty_like(x), torch.empty(K * Co, device="cuda", dtype=tdt), torch.empty(Co, device="cuda", dtype=tdt)
        fwd, bwd = _lib.conv2d(dt)
        for mode, label in ((1, "direct"), (0, "reference_calls")):
            ms_f = time_launches(torch, lambda: fwd(ctypes.byref(conv), mode, x.data_ptr(), w.data_ptr(), bias.data_ptr(), cols.data_ptr(), ws.data_ptr(),
                                                    out.data_ptr()), iters, 2)
            row_f = {"case": f"conv2d_forward_{dt}/{label}", "ms": round(ms_f, 4), "gemm_tflops_equiv": round(flop / ms_f / 1e9, 1),
                     "what": "im2col + product + bias add"}
            if verify and mode == 1:
                row_f["verified"] = bool(verify_conv_forward(torch, dt, cv, x, w, bias, out))
            ms_b = time_launches(torch, lambda: bwd(ctypes.byref(conv), mode, go.data_ptr(), w.data_ptr(), cols.data_ptr(), ws.data_ptr(), gx.data_ptr(),
                                                    gw.data_ptr(), gb.data_ptr()), iters, 2)
            row_b = {"case": f"conv2d_backward_{dt}/{label}", "ms": round(ms_b, 4), "gemm_tflops_equiv": round(2 * flop / ms_b / 1e9, 1),
                     "what": "grad input (product + col2im), grad weight (product), grad bias (three sums)"}
            if verify and mode == 1:
                row_b["verified"] = bool(verify_conv_weight_grad(torch, dt, cv, x, go, gw))
            rows += [row_f, row_b]
        del x, w, bias, go, cols, ws, out, gx, gw, gb
        torch.cuda.empty_cache()
        # the three products of the literal call sequence, alone: [B*P, K] x [K, Co], [B*P, Co] x [Co, K], [K, B*P] x [B*P, Co]
        M = B * P
        kern = "tc_gemm_kernel" if dt == "bf16" else "tc_gemm_f32_kernel"
        rows.append(gemm_row(torch, lib_mod, f"conv_gemm_forward_{dt}", dt, M, Co, K, "k", "k", peaks["bf16_tflops"], iters, verify, kern))
        rows.append(gemm_row(torch, lib_mod, f"conv_gemm_grad_cols_{dt}", dt, M, K, Co, "k", "mn", peaks["bf16_tflops"], iters, verify, kern))
        rows.append(gemm_row(torch, lib_mod, f"conv_gemm_grad_weight_{dt}", dt, K, Co, M, "mn", "mn", peaks["bf16_tflops"], iters, verify, kern))
        torch.cuda.empty_cache()
    return rows


def verify_conv_forward(torch, dt, cv, x, w, bias, out):
    """Direct form: sampled output positions against a float64 convolution evaluated at those positions only."""
    B, C, H, W, Co, k, p = cv["B"], cv["C"], cv["H"], cv["W"], cv["Co"], cv["k"], cv["p"]
    xs = x.view(B, C, H, W).double()
    wd = w.view(Co, C, k, k).double()
    bd = bias.double()
    o = out.view(B, Co, H, W)
    rng = np.random.default_rng(5)
    ok = True
    for _ in range(24):
        b_, y_, x_ = int(rng.integers(0, B)), int(rng.choice([0, 1, H // 2, H - 1])), int(rng.choice([0, 1, W // 2, W - 1]))
        acc = bd.clone()
        for i in range(k):
            for j in range(k):
                yy, xx = y_ - p + i, x_ - p + j
                if 0 <= yy < H and 0 <= xx < W:
                    acc += wd[:, :, i, j] @ xs[b_, :, yy, xx]
        got = o[b_, :, y_, x_].double()
        rel = 1e-4 if dt == "f32" else 2e-2
        ok = ok and bool(torch.all((got - acc).abs() <= rel * torch.maximum(acc.abs(), torch.ones_like(acc))).item())
    return ok


def verify_conv_weight_grad(torch, dt, cv, x, go, gw):
    """Direct form: sampled weight-gradient entries against float64 sums over the whole batch and image."""
    B, C, H, W, Co, k, p = cv["B"], cv["C"], cv["H"], cv["W"], cv["Co"], cv["k"], cv["p"]
    xs = x.view(B, C, H, W)
    g = go.view(B, Co, H, W)
    G = gw.view(Co, C, k, k)
    rng = np.random.default_rng(6)
    ok = True
    for _ in range(12):
        co, ci, i, j = int(rng.integers(0, Co)), int(rng.integers(0, C)), int(rng.integers(0, k)), int(rng.integers(0, k))
        y0, y1 = max(0, p - i), min(H, H + p - i)   # output rows whose input row y - p + i is inside the image
        x0, x1 = max(0, p - j), min(W, W + p - j)
        ref = (g[:, co, y0:y1, x0:x1].double() * xs[:, ci, y0 - p + i:y1 - p + i, x0 - p + j:x1 - p + j].double()).sum()
        got = G[co, ci, i, j].double()
        rel = 1e-4 if dt == "f32" else 2e-2
        ok = ok and bool(((got - ref).abs() <= rel * max(abs(float(ref)), (B * H * W) ** 0.5)).item())
    return ok


# ---------------------------------------------------------------------------------------
# data movement either side of the ops: dtype casts and contiguous() on the device
# ---------------------------------------------------------------------------------------
def movement_rows(torch, lib_mod, peaks, iters, small=False):
    n = (1 << 26) if small else (1 << 28)
    R = 8192 if small else 16384
    rows = []
    src32 = make_inputs(torch, "f32", n, 31)
    src16 = src32.bfloat16()
    for frm, to, src in (("f32", "bf16", src32), ("bf16", "f32", src16), ("f32", "f16", src32)):
        out = torch.empty(n, dtype=torch_dtype(to), device="cuda")
        fn = lib_mod.cast(frm, to)
        ms = time_launches(torch, lambda: fn(SZ(n), src.data_ptr(), out.data_ptr()), iters, 3)
        nbytes = n * (src.element_size() + out.element_size())
        ref = src.to(torch_dtype(to))
        rows.append({"case": f"cast_{frm}_{to}", "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "bytes": nbytes,
                     "frac": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4), "verified": bool(torch.equal(out, ref))})
        del out, ref
    for dt, src in (("f32", src32), ("bf16", src16)):
        out = torch.empty(n, dtype=src.dtype, device="cuda")
        meta = np.array([R, n // R, 1, R, 0], dtype=np.uint64)  # the transposed view of a dense [n / R, R] matrix
        fn = lib_mod.contiguous(dt)
        ms = time_launches(torch, lambda: fn(SZ(n), SZ(2), meta.ctypes.data, src.data_ptr(), out.data_ptr()), iters, 3)
        nbytes = 2 * n * src.element_size()
        ok = bool(torch.equal(out.view(R, n // R), src.view(n // R, R).t()))
        rows.append({"case": f"contiguous_{dt}/transposed", "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "bytes": nbytes,
                     "frac": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4), "verified": ok})
        del out
    return rows


# ---------------------------------------------------------------------------------------
# BASELINE config 1: the README training example, every op through the reference's dispatch pattern
# ---------------------------------------------------------------------------------------
class OracleEngine:
    """The engine interface of maidenx_b200.readme_example on the CPU oracle (numpy buffers, host metadata)."""
    name = "oracle"

    def upload(self, arr):
        return np.ascontiguousarray(arr, dtype=np.float32).copy()

    def empty(self, count):
        return np.empty(max(count, 1), np.float32)

    def free(self, buf):
        pass

    def ptr(self, buf):
        return buf.ctypes.data

    def call(self, op, metadata, *args):
        from oracle import binding
        m = np.asarray(metadata, dtype=np.uint64)
        binding.op(op, "f32")(*[m.ctypes.data if (isinstance(a, str) and a == "META") else a for a in args])

    def read(self, buf, count):
        return buf[:count].copy()


def config1_row(torch, lib, steps=200, with_cpu=True):
    """Steps per second of the README example (Linear(3 -> 1) + MSE + SGD, f32, 10000 x 3; 17 op calls per step, each
    with its metadata upload and every output a cuda_malloc'ed buffer), with and without the caching allocator, and the
    same sequence on the CPU oracle.  Host wall clock: the workload is dispatch-bound by construction."""
    from maidenx_b200 import readme_example as E
    row = {"case": "readme_example_linear3x1_f32", "ops_per_step": E.OPS_PER_STEP, "steps": steps}
    for label, on in (("cached_allocator", 1), ("cuda_malloc_free", 0)):
        lib.mx_set_small_pool(on)
        E.train(E.CudaEngine(), 20)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        losses, W, b = E.train(E.CudaEngine(), steps)
        torch.cuda.synchronize()
        dt_s = time.perf_counter() - t0
        row[label + "_steps_per_s"] = round(steps / dt_s, 1)
        row[label + "_us_per_op"] = round(dt_s / steps / E.OPS_PER_STEP * 1e6, 2)
        row[label + "_loss"] = losses[-1]
    lib.mx_set_small_pool(1)
    if with_cpu:
        from oracle import binding
        binding.load()
        binding.set_num_threads(os.cpu_count() or 1)
        binding.set_reduce_parallel(True)  # the reference's reductions: a parallel loop with one lock per output element
        t0 = time.perf_counter()
        cl, cW, cb = E.train(OracleEngine(), steps)
        dt_s = time.perf_counter() - t0
        row["cpu_steps_per_s"] = round(steps / dt_s, 1)
        row["cpu_cores"] = binding.max_threads()
        row["verified"] = bool(np.allclose(losses, cl, rtol=1e-4) and np.allclose(W, cW, rtol=1e-4, atol=1e-6) and np.allclose(b, cb, rtol=1e-4, atol=1e-6))
    return row

# ---------------------------------------------------------------------------------------
# workload: data-parallel MLP training step (the headline at every N)
# ---------------------------------------------------------------------------------------
MLP_LAYERS, MLP_DIM, MLP_GLOBAL_BATCH, MLP_LR = 4, 8192, 16384, 1e-3
MLP_GEMMS_PER_STEP = 3 * MLP_LAYERS - 1       # dX of the first layer is not needed and not computed
# kernels launched per step: 11 GEMMs (the 4 forward ones carry the bias add and GELU in their epilogue) + 2 (mse,
# mse finish) + 3 gelu backward + 4 bias-gradient sums (partials folded inside the same launch) + 8 SGD updates (weights
# and bias per layer; on a side stream at N = 1); with the NVLink exchange the 8 SGD launches become
# 4 x (barrier, fused reduce + update, barrier)
MLP_KERNELS_PER_STEP = MLP_GEMMS_PER_STEP + 2 + (MLP_LAYERS - 1) + MLP_LAYERS + 2 * MLP_LAYERS


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


def verify_mlp(torch, mlp, x, y, local_batch, rows=4):
    """Before any weight update: (a) the network output of a few batch rows against the same network composed from
    CPU-oracle ops (oracle/mlp_reference.py, wide accumulation) with THIS engine's weights, (b) the loss the engine
    reports against a float64 mean over its own full output."""
    from maidenx_b200.mlp import _as_tensor
    from oracle import binding, mlp_reference
    binding.load()
    binding.set_num_threads(os.cpu_count() or 1)
    n2 = MLP_DIM * MLP_DIM
    W = [to_store(_as_tensor(torch, mlp.ptr("weight", l), n2, torch.bfloat16)) for l in range(MLP_LAYERS)]
    from maidenx_b200 import dtypes as D
    bias = []
    for l in range(MLP_LAYERS):
        raw = torch.as_tensor(_F32Array(mlp.ptr("master_bias", l), 1), device="cuda")
        bias.append(D.encode(raw.cpu().numpy(), D.BF16))
    mlp.forward(x.data_ptr())
    mlp.loss_backward(y.data_ptr())
    torch.cuda.synchronize()
    out = _as_tensor(torch, mlp.ptr("output"), local_batch * MLP_DIM, torch.bfloat16).view(local_batch, MLP_DIM)
    r = sample_rows(local_batch, rows, 3)
    idx = torch.as_tensor(r, device="cuda")
    ref_net = mlp_reference.CpuMlp(MLP_LAYERS, MLP_DIM, len(r), "bf16", W, bias)
    binding.set_wide(True)
    try:
        ref_net.gradients(to_store(x[idx]), to_store(y[idx]))
    finally:
        binding.set_wide(False)
    ref_out = ref_net.last_output
    scale = float(np.sqrt(np.mean(decode(ref_out, "bf16") ** 2)))
    rows_ok = close(to_store(out[idx]), ref_out, "bf16", 2e-2, scale)
    loss64 = float(((out.double() - y.double()) ** 2).mean().item())
    loss_ok = abs(mlp.loss() - loss64) <= 1e-4 * abs(loss64)
    return bool(rows_ok), bool(loss_ok)


class _F32Array:
    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}


def e2e_mlp(torch, lib, mlp, x, y, dist, world, steps, warm):
    """The same step fed from pinned host memory: every step copies its shard's inputs host -> device and reads the
    loss back.  The copies of step i + 1 run on a copy stream into the second of two device buffers while step i
    computes (an input pipeline: the user-facing loop of maidenx_b200.mlp.InputPipeline)."""
    from maidenx_b200.mlp import InputPipeline, LossReader
    hx, hy = x.cpu().pin_memory(), y.cpu().pin_memory()
    nbytes = x.numel() * x.element_size()
    pipe = InputPipeline(torch, x, y)
    reader = LossReader(torch, mlp)
    losses = []

    def run(n):
        pipe.prefetch(hx, hy)
        for i in range(n):
            xb, yb = pipe.next_batch()          # the compute stream now waits for this batch's copies
            if i + 1 < n:
                pipe.prefetch(hx, hy)           # next batch: copies overlap this step
            mlp.train_step(xb.data_ptr(), yb.data_ptr(), MLP_LR, torch, dist, world)
            pipe.release()                      # the buffers may be overwritten once this step's kernels are done
            prev = reader.after_step()          # this step's loss copy is queued; the previous step's loss is on the host now
            if prev is not None:
                losses.append(prev)
        losses.append(reader.last())            # the last step's loss: read inside the timed region too

    run(warm)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    del losses[:]
    t0 = time.perf_counter()
    run(steps)
    torch.cuda.synchronize()
    dt_s = (time.perf_counter() - t0) / steps
    if world > 1:
        t = torch.tensor([dt_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt_s = float(t.item())
    # the feed alone: the same pinned -> device copies with no compute beside them, every rank at the same time.  When this
    # rate is below what the device-resident step consumes, the host link (not the kernels, not the exchange) bounds e2e.
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(4):
        pipe.bufs[0][0].copy_(hx, non_blocking=True)
        pipe.bufs[0][1].copy_(hy, non_blocking=True)
    torch.cuda.synchronize()
    copy_s = (time.perf_counter() - t0) / 4
    if world > 1:
        t = torch.tensor([copy_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        copy_s = float(t.item())
    return {"value": round(MLP_GLOBAL_BATCH / dt_s, 1), "unit": "samples/s", "h2d_bytes_per_step": 2 * nbytes * world, "d2h_bytes_per_step": 4 * world,
            "steps": steps, "ms_per_step": round(dt_s * 1e3, 3), "loss": losses[-1], "losses_read": len(losses),
            "pipeline": "double-buffered: host->device copies of step i+1 on a copy stream while step i computes; every step's loss is copied "
                        "to pinned host memory on its own stream and collected by the host one step later (maidenx_b200.mlp.LossReader)",
            "h2d_gbs_per_rank_achieved": round(2 * nbytes / dt_s / 1e9, 1),
            "h2d_copy_only": {"ms_per_step_worth": round(copy_s * 1e3, 3), "gbs_per_rank": round(2 * nbytes / copy_s / 1e9, 1),
                              "gbs_all_ranks": round(2 * nbytes * world / copy_s / 1e9, 1),
                              "what": "the step's input copies alone (pinned host memory, all ranks at once, slowest rank): the floor under any e2e step time"}}


def cpu_mlp_once(sample_batch, steps=1):
    """One size of the CPU arm: the same model and step composed from the CPU port of the reference's backend (full
    4 x 8192^2 weights, `sample_batch` rows); best seconds per step."""
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
    return best, binding.max_threads()


def cpu_mlp(sizes=(4, 16), steps=1):
    """The CPU arm at two sample sizes.  A step costs fixed + per_row * rows (the weight update and the weight-sized
    passes do not depend on the batch); both coefficients come from the two measurements, and the full-batch figure
    derived from them is reported as DERIVED next to the measured ones.  `value` is the measured throughput of the
    larger sample."""
    t = []
    cores = 1
    for s in sizes:
        sec, cores = cpu_mlp_once(s, steps)
        t.append(sec)
    per_row = max((t[1] - t[0]) / (sizes[1] - sizes[0]), 1e-9)
    fixed = max(t[0] - per_row * sizes[0], 0.0)
    full = fixed + per_row * MLP_GLOBAL_BATCH
    return {"value": round(sizes[1] / t[1], 3), "unit": "samples/s", "cores": cores, "kind": "port",
            "sample": f"one full training step (4 x Linear(8192->8192), GELU, MSE, SGD, bf16; weights and update at full size) on "
                      f"{sizes[0]} rows ({t[0]:.1f} s) and on {sizes[1]} rows ({t[1]:.1f} s) of the 16384",
            "measured": [{"rows": s, "seconds_per_step": round(x, 2), "samples_per_s": round(s / x, 3)} for s, x in zip(sizes, t)],
            "fit": {"fixed_seconds_per_step": round(fixed, 2), "seconds_per_row": round(per_row, 4)},
            "derived_full_batch": {"seconds_per_step": round(full, 1), "samples_per_s": round(MLP_GLOBAL_BATCH / full, 3),
                                   "note": "DERIVED from the fit, not measured: fixed + 16384 * per_row"}}, t[1]


def reference_arm(args):
    """`--impl reference`: the reference's own CPU implementation of the path is a Rust crate that cannot be
    built here, so this arm times its CPU port (the oracle) on all host cores: the same model and step on a
    bounded sample of the batch.  Rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps = max(1, min(args.steps, 2))
    cb, sec = cpu_mlp((4, 16), steps=steps)
    line = {"metric": "mlp_train_samples_per_s", "value": cb["value"], "unit": "samples/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": 0, "ms_per_step": round(sec * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 (element-type accumulation, as the reference's CPU backend)", "data": "synthetic", "impl": "reference",
            "config": {"workload": "MLP data-parallel training step: 4 x Linear(8192->8192) + GELU, MSE, SGD lr=1e-3",
                       "global_batch": MLP_GLOBAL_BATCH, "sample_rows": 16,
                       "note": "a step is the full-size model on a 16-row sample of the batch; see cpu_baseline.derived_full_batch for the full-batch figure the fit gives"},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def summarize(rows, key="frac"):
    vals = [(r[key], r["case"]) for r in rows if key in r]
    if not vals:
        return {}
    fr = sorted(v for v, _ in vals)
    worst = min(vals)
    out = {"cases": len(vals), "min_frac": fr[0], "median_frac": fr[len(fr) // 2], "worst_case": worst[1],
           "at_or_above_80pct_of_measured": sum(1 for v in fr if v >= 0.8)}
    if any("verified" in r for r in rows):
        out["verified"] = sum(1 for r in rows if r.get("verified"))
        out["verify_failed"] = [r["case"] for r in rows if r.get("verified") is False]
    cpu = [r["cpu_gbs"] for r in rows if "cpu_gbs" in r]
    if cpu:
        out["cpu_gbs_median"] = sorted(cpu)[len(cpu) // 2]
    return out


# ---------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweeps", action="store_true", help="skip the per-case tables (elementwise, reductions, conv, products, movement)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true", help="skip every CPU-oracle timing")
    ap.add_argument("--no-verify", action="store_true", help="skip the output checks against the CPU oracle")
    ap.add_argument("--global-batch", type=int, default=None,
                    help="tuning aid: another global batch than the benchmark's 16384 (the JSON line says so; not a headline number)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "multimem-exclusive", "copy", "multimem", "peer", "nccl"],
                    help="N > 1: how gradients are exchanged (auto: the library's NVLink kernels, NCCL if symmetric memory is unavailable)")
    ap.add_argument("--exchange-sms", type=int, default=8, help="multimem-exclusive: SMs given to the exchange kernel")
    ap.add_argument("--cta-group", type=int, default=1, choices=[1, 2], help="bf16 / f16 tensor-core products: 1 = one CTA per tile (default), 2 = pairs of CTAs share the B tile (same rate on a power-capped B200)")
    ap.add_argument("--group-m", type=int, default=0, help="tuning aid: row-tiles per column sweep of the GEMM's tile order (0 = the library's default)")
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
    lib.mx_set_gemm_cta_group(args.cta_group)
    if args.group_m:
        lib.mx_debug_set_gemm_group_m(args.group_m)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    verify = not args.no_verify

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
    verified = {}
    if verify and world == 1:
        rows_ok, loss_ok = verify_mlp(torch, mlp, x, y, local_batch)
        verified["mlp_output_rows_vs_oracle"] = rows_ok
        verified["mlp_loss_vs_f64"] = loss_ok

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
    if world > 1 and verify:
        # data parallelism keeps replicas in step: after the timed steps every rank must hold bit-identical weights
        from maidenx_b200.mlp import _as_tensor
        sums = []
        for l in range(MLP_LAYERS):
            w = _as_tensor(torch, mlp.ptr("weight", l), MLP_DIM * MLP_DIM, torch.bfloat16).view(torch.int16).to(torch.int64)
            sums.append((w * (torch.arange(w.numel(), device="cuda") % 8191 + 1)).sum())
        mine = torch.stack(sums)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        verified["weights_bit_identical_across_ranks"] = bool(torch.equal(lo, hi))
    if hasattr(mlp, "status") and mlp.status() != 0:
        raise RuntimeError(f"a cross-rank barrier gave up waiting for rank {mlp.status() - 1}")
    lib.mx_device_synchronize()
    if lib.mx_last_error():
        raise RuntimeError(f"op library reported status {lib.mx_last_error()} at {lib.mx_last_error_where().decode()}")
    value = MLP_GLOBAL_BATCH / (ms_step / 1e3)

    # the dominant kernel alone, live, on this rank's shapes: bursts, each with the SM clock seen while it ran
    probe = ClockProbe(local_rank)
    bursts, gemm_bufs = time_gemm_bursts(torch, lib_mod, probe, local_batch, MLP_DIM, MLP_DIM)
    gemm_flops = 2.0 * local_batch * MLP_DIM * MLP_DIM
    if verify and rank == 0:
        verified["gemm_rows_vs_oracle"] = bool(verify_gemm(torch, "bf16", local_batch, MLP_DIM, MLP_DIM, *gemm_bufs))
    same_method = gemm_same_method_as_peak(torch, lib_mod, local_batch, MLP_DIM, MLP_DIM, gemm_bufs) if rank == 0 else None
    del gemm_bufs
    e2e = None if args.no_e2e else e2e_mlp(torch, lib, mlp, x, y, dist, world, steps=6, warm=2)
    clocks = sampler.stop()

    sweeps_out, roofline, cpu = {}, None, None
    if rank == 0:
        tf = sorted(b["tflops"] for b in bursts)
        med = tf[len(tf) // 2]
        gemm_ms = gemm_flops / med / 1e9
        prof = profiled_traffic("tc_gemm_kernel", "8192x4096x8192")
        traffic = int((prof["read"] + prof["write"]) / prof["work"] * gemm_flops) if prof else None
        roofline = {"bound": "tensor", "kernel": "tc_gemm_kernel", "achieved": round(med, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": round(med / peaks["bf16_tflops"], 4), "peak_source": peaks["source"] + " (burst: kernel timed alone)",
                    "frac_of_nominal_2250": round(med / NOMINAL_BF16_TFLOPS, 4),
                    "launch_shape": f"[{local_batch},{MLP_DIM}] x [{MLP_DIM},{MLP_DIM}]^T bf16", "flops_per_launch": gemm_flops,
                    "ms_per_launch": round(gemm_ms, 4), "bursts": bursts, "spread_tflops": [tf[0], tf[-1]],
                    "timing": f"median of {len(bursts)} bursts of 12 back-to-back launches after 5 warm-up launches",
                    "same_method_as_peak": same_method,
                    "frac_best_of_10": round(same_method["tc_gemm_kernel"]["best_of_10_tflops"] / peaks["bf16_tflops"], 4),
                    "traffic": traffic,
                    "traffic_source": "ncu capture at 8192x4096x8192 (profiles/dram_traffic_per_launch.md) scaled by flops: same K, tile shape and tile order" if prof else None,
                    "step_gemm_share": round(MLP_GEMMS_PER_STEP * gemm_ms / ms_step, 3),
                    "step_tflops": round(mlp_flops(local_batch) * world / ms_step / 1e9, 1),
                    "step_frac_of_sustained": round(mlp_flops(local_batch) / ms_step / 1e9 / peaks["bf16_tflops_sustained"], 4)}
    del mlp, x, y
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_sweeps:
        with_cpu = not args.no_cpu
        groups = (("elementwise", sweeps.elementwise_cases(), sweeps.elementwise_cases(1024, 16384), (1, 101), "uniform"),
                  ("reduction", sweeps.reduction_cases(), sweeps.reduction_cases(512, 16384, (4, 512, 4096)), (3, 103), "normal"),
                  ("conv", sweeps.conv_cases(), sweeps.conv_cases(N=2), (10, 110), "normal"),
                  ("extras", sweeps.extras_cases(), sweeps.extras_cases(rows=512, N=2), (12, 112), "normal"))
        cores = None
        for name, cases, small_cases, seeds, kind in groups:
            rows, cores_g = run_sweep_group(torch, lib_mod, cases, small_cases, 10, 3, seeds, kind, peaks, verify, with_cpu)
            cores = cores_g or cores
            sweeps_out[name] = rows
        it = 5
        pk = peaks["bf16_tflops"]
        sweeps_out["matmul"] = [
            gemm_row(torch, lib_mod, "matmul_bf16/16384x8192x8192/nt", "bf16", 16384, 8192, 8192, "k", "k", pk, it, False, "tc_gemm_kernel"),
            gemm_row(torch, lib_mod, "matmul_f16/16384x8192x8192/nt", "f16", 16384, 8192, 8192, "k", "k", pk, it, verify, "tc_gemm_kernel"),
            gemm_row(torch, lib_mod, "matmul_f32/16384x8192x8192/nt", "f32", 16384, 8192, 8192, "k", "k", pk, 3, verify, "tc_gemm_f32_kernel (split tf32)"),
            gemm_row(torch, lib_mod, "matmul_f32/4096x4098x4096/nn", "f32", 4096, 4098, 4096, "k", "mn", pk, 3, verify, "matmul_simt_kernel (row pitch not a multiple of 16 bytes)"),
        ]
        sweeps_out["conv2d_layer"] = conv_rows(torch, lib_mod, peaks, 3, verify)
        sweeps_out["movement"] = movement_rows(torch, lib_mod, peaks, 10)
        sweeps_out["config1"] = config1_row(torch, lib, with_cpu=with_cpu)
        hbm_rows = sweeps_out["elementwise"] + sweeps_out["reduction"] + sweeps_out["conv"] + sweeps_out["movement"]
        ew = sweeps_out["elementwise"]
        summary = {g: summarize(sweeps_out[g]) for g in ("elementwise", "reduction", "conv", "movement", "extras")}
        summary["all_hbm_cases"] = summarize(hbm_rows)
        summary["all_hbm_cases"]["min_frac_of_nominal_8000"] = round(min(r["gbs"] for r in hbm_rows) / NOMINAL_HBM_GBS, 4)
        summary["all_hbm_cases"]["median_frac_of_nominal_8000"] = round(sorted(r["gbs"] for r in hbm_rows)[len(hbm_rows) // 2] / NOMINAL_HBM_GBS, 4)
        summary["elementwise_aggregate_gbs"] = round(sum(r["bytes"] for r in ew) / sum(r["ms"] for r in ew) / 1e6, 1)
        summary["peak_gbs"], summary["peak_source"], summary["cpu_cores"] = peaks["hbm_gbs"], peaks["source"], cores
        summary["products_tflops"] = {r["case"]: r["tflops"] for r in sweeps_out["matmul"] + sweeps_out["conv2d_layer"] if "tflops" in r}
        summary["conv2d_layer_ms"] = {r["case"]: r["ms"] for r in sweeps_out["conv2d_layer"] if "what" in r}
        c1 = sweeps_out["config1"]
        summary["config1_steps_per_s"] = {k: c1.get(k) for k in ("cached_allocator_steps_per_s", "cuda_malloc_free_steps_per_s", "cpu_steps_per_s")}
        every = [r for g in ("elementwise", "reduction", "conv", "matmul", "conv2d_layer", "movement", "extras") for r in sweeps_out[g]] + [c1]
        verified["sweep_cases_checked"] = sum(1 for r in every if "verified" in r)
        verified["sweep_cases_failed"] = [r["case"] for r in every if r.get("verified") is False]
        roofline["sweeps"] = summary
        if lib.mx_last_error():
            raise RuntimeError(f"op library reported status {lib.mx_last_error()} at {lib.mx_last_error_where().decode()}")
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = cpu_mlp((4, 16))

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        exch = mlp_exchange in ("multimem", "multimem-exclusive", "peer", "copy")
        line = {"metric": "mlp_train_samples_per_s", "value": round(value, 1), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16 (f32 accumulate, f32 master weights)",
                "data": "synthetic (seeded N(0,1) inputs and targets, Kaiming-uniform weights U(-1/sqrt(8192), 1/sqrt(8192)))",
                "config": {"workload": "MLP data-parallel training step: 4 x Linear(8192->8192) + GELU, MSE, SGD lr=1e-3", "global_batch": MLP_GLOBAL_BATCH,
                           "per_gpu_batch": local_batch, "parallelism": f"dp{world}", "allreduce": EXCHANGE_TEXT[mlp_exchange],
                           "l2": "per-step working set (weights 0.5 GB + activations 2 GB per GPU at N=1) far exceeds the 126 MB L2; sweep inputs are 0.5-2 GB",
                           "verified": verified if verify else "skipped (--no-verify)"},
                "loss": loss, "clocks": clocks, "gpu_launches": (MLP_KERNELS_PER_STEP + (3 * MLP_LAYERS - 2 * MLP_LAYERS if exch else 0)) * args.steps,
                "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu, "sweeps": sweeps_out}
        print(json.dumps(line))


def run_only_case(torch, lib_mod, args):
    """Launch one sweep case a few times (for ncu captures of a single kernel)."""
    peaks = measured_peaks()
    if args.small:
        groups = sweeps.elementwise_cases(8192, 8192) + sweeps.reduction_cases(4096, 16384, (16, 512, 4096)) + sweeps.conv_cases(N=16) + sweeps.extras_cases(rows=4096, N=16)
    else:
        groups = sweeps.elementwise_cases() + sweeps.reduction_cases() + sweeps.conv_cases() + sweeps.extras_cases()
    if args.only_case.startswith("library_gemm_"):
        # library_gemm_<bf16|f16>[_<MxNxK>]: torch.matmul (the library GEMM) on the operands gemm_<dt> uses - a comparison point
        # for profiles, never the product path
        parts = args.only_case.split("_")
        dt = parts[2]
        M, N, K = (8192, 4096, 8192) if args.small else (MLP_GLOBAL_BATCH, MLP_DIM, MLP_DIM)
        if len(parts) > 3:
            M, N, K = (int(v) for v in parts[3].split("x"))
        a, b, c, _ = gemm_operands(torch, dt, M, N, K)
        ms = time_launches(torch, lambda: torch.matmul(a, b.t(), out=c), max(1, args.steps), max(0, args.warmup))
        print(json.dumps({"case": args.only_case, "shape": [M, N, K], "ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)}))
        return
    if args.only_case.startswith("gemm_"):
        # gemm_<bf16|f16|f32>[_<MxNxK>[_<nt|nn|tn|tt>]]: a product alone; default x . W^T of one MLP layer; --small: 8192 x 4096 x 8192
        parts = args.only_case.split("_")
        dt = parts[1]
        M, N, K = (8192, 4096, 8192) if args.small else (MLP_GLOBAL_BATCH, MLP_DIM, MLP_DIM)
        if len(parts) > 2:
            M, N, K = (int(v) for v in parts[2].split("x"))
        lay = parts[3] if len(parts) > 3 else "nt"
        a_major, b_major = ("k" if lay[0] == "n" else "mn"), ("k" if lay[1] == "t" else "mn")
        a, b, c, meta = gemm_operands(torch, dt, M, N, K, a_major, b_major)
        f = lib_mod.op("matmul", dt)
        ms = time_launches(torch, lambda: f(SZ(M * N), meta.ctypes.data, a.data_ptr(), b.data_ptr(), c.data_ptr()), max(1, args.steps), max(0, args.warmup))
        lib_mod.load().mx_device_synchronize()
        print(json.dumps({"case": args.only_case, "shape": [M, N, K], "ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1),
                          "status": lib_mod.load().mx_last_error()}))
        return
    if args.only_case == "conv2d_layer":
        print(json.dumps(conv_rows(torch, lib_mod, peaks, max(1, args.steps), not args.no_verify, small=args.small)))
        return
    if args.only_case == "movement":
        print(json.dumps(movement_rows(torch, lib_mod, peaks, max(1, args.steps), small=args.small)))
        return
    if args.only_case == "config1":
        print(json.dumps(config1_row(torch, lib_mod.load(), with_cpu=not args.no_cpu)))
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
    res = {"case": c.name, "ms": round(ms, 4), "gbs": round(c.bytes / ms / 1e6, 1), "status": lib_mod.load().mx_last_error()}
    if not args.no_verify:
        res["verified"] = bool(verify_case(torch, c, a, b, out))
    print(json.dumps(res))


if __name__ == "__main__":
    main()
