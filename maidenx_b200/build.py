"""Builds libmaidenx_cuda.so in-tree with nvcc for sm_100a.

The kernels are written for Blackwell only: a single -gencode for compute_100a/sm_100a,
no fallback architectures.  Family sources (binary.cu, unary.cu, ...) are compiled once
per dtype so that the ~30 translation units build in parallel; objects are cached under
csrc/build/ and rebuilt when any source or header is newer.

Usage:  python -m maidenx_b200.build [--force] [--jobs N] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD = CSRC / "build"
LIB_PATH = PKG_DIR / "libmaidenx_cuda.so"

# suffix -> class id (see abi_common.cuh)
DTYPES = {
    "bf16": 1, "f16": 1, "f32": 1, "f64": 1,
    "u8": 2, "u16": 2, "u32": 2, "u64": 2,
    "i8": 3, "i16": 3, "i32": 3, "i64": 3,
    "bool": 4,
}
ARITH = [d for d in DTYPES if d != "bool"]
FLOATS = ["bf16", "f16", "f32", "f64"]

# source file -> dtypes it is compiled for (None = compiled once, not per dtype)
PER_DTYPE_SOURCES = {
    "binary.cu": list(DTYPES),
    "unary.cu": list(DTYPES),
}
SINGLE_SOURCES = ["runtime.cu", "ew_plan.cu"]


def _register_optional():
    """Families added as the library grows; only listed when the file exists."""
    for name, dts in (("reduction.cu", ARITH), ("matmul_simt.cu", ARITH), ("conv.cu", FLOATS), ("extras.cu", ARITH)):
        if (CSRC / name).exists():
            PER_DTYPE_SOURCES[name] = dts
    for name in ("reduce_plan.cu", "matmul_plan.cu", "matmul_tc.cu", "matmul_tc2.cu", "matmul_tc_f32.cu", "fused.cu", "mlp.cu", "noalloc.cu", "dp_sync.cu", "cast.cu", "conv2d_layer.cu"):
        if (CSRC / name).exists() and name not in SINGLE_SOURCES:
            SINGLE_SOURCES.append(name)


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the op library cannot be built")


def base_flags() -> list[str]:
    return [
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        "--expt-relaxed-constexpr",
        # No implicit FMA contraction: elementwise results then match the CPU backend's
        # separately-rounded multiplies and adds bit for bit.  Kernels that want FMA
        # (matmul) ask for it explicitly with fmaf / tensor cores.
        "-fmad=false",
        "-Xcompiler", "-fPIC",
        # ~2700 small kernels with line info: compress the embedded cubins (4x smaller .so).
        "-Xfatbin=-compress-all",
        # nvcc honours the CXX/CC environment only through -ccbin; pin the system g++.
        "-ccbin", "/usr/bin/g++",
        "-I", str(INCLUDE), "-I", str(CSRC),
    ]


def _newest_header_mtime() -> float:
    m = 0.0
    for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]:
        m = max(m, p.stat().st_mtime)
    return m


def _jobs() -> list[tuple[Path, Path, list[str]]]:
    _register_optional()
    jobs = []
    for src in SINGLE_SOURCES:
        jobs.append((CSRC / src, BUILD / (Path(src).stem + ".o"), []))
    for src, dts in PER_DTYPE_SOURCES.items():
        for dt in dts:
            jobs.append((CSRC / src, BUILD / f"{Path(src).stem}_{dt}.o", [f"-DMX_T={dt}", f"-DMX_TCLASS={DTYPES[dt]}"]))
    return jobs


def build(force: bool = False, jobs: int | None = None, verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = nvcc_path()
    BUILD.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    todo = []
    all_objs = []
    for src, obj, defs in _jobs():
        all_objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            todo.append((src, obj, defs))

    def run(job):
        src, obj, defs = job
        cmd = [nvcc, *base_flags(), *defs, "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name} {' '.join(defs)}:\n{r.stdout}\n{r.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(f"[build] {obj.name}\n{r.stderr if ptxas_info else ''}")
        return obj

    if todo:
        nthreads = jobs or max(1, (os.cpu_count() or 4))
        with ThreadPoolExecutor(max_workers=nthreads) as ex:
            list(ex.map(run, todo))
    if todo or not LIB_PATH.exists() or force:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "/usr/bin/g++",
               "-Xcompiler", "-fPIC", "-o", str(LIB_PATH), *map(str, all_objs), "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="pass -Xptxas -v (registers, spills, shared memory)")
    a = ap.parse_args(argv)
    p = build(force=a.force, jobs=a.jobs, verbose=a.verbose, ptxas_info=a.ptxas_info)
    print(p)


if __name__ == "__main__":
    main()
