"""ctypes binding of the CPU oracle.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the
smoke check and by the benchmark's CPU-baseline leg; nothing in the product imports it."""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libmaidenx_cpu_oracle.so"

sys.path.insert(0, str(HERE.parent))
from maidenx_b200 import _signatures as sig  # noqa: E402  (signature table only; no CUDA involved)

_lib = None
_ops = None


def build(force: bool = False) -> Path:
    src_m = max((HERE / n).stat().st_mtime for n in ("maidenx_cpu_oracle.cpp", "half_types.h", "Makefile"))
    if force or not LIB.exists() or LIB.stat().st_mtime < src_m:
        env = dict(os.environ)
        env.pop("CXXFLAGS", None)
        subprocess.run(["make", "-C", str(HERE), "-s"], check=True, env=env)
    return LIB


def load() -> ctypes.CDLL:
    global _lib, _ops
    if _lib is None:
        build()
        lib = ctypes.CDLL(str(LIB))
        lib.oracle_set_wide.argtypes = [ctypes.c_int]
        lib.oracle_set_reduce_parallel.argtypes = [ctypes.c_int]
        lib.oracle_set_num_threads.argtypes = [ctypes.c_int]
        lib.oracle_get_max_threads.restype = ctypes.c_int
        _ops = sig.bind(lib, "")
        _lib = lib
    return _lib


def op(name: str, dtype_name: str):
    load()
    return _ops[(name, dtype_name)]


def cast(from_name: str, to_name: str):
    """cast_<from>_<to>(num_els, in, out): the reference's host-side dtype conversion, element by element."""
    fn = getattr(load(), f"cast_{from_name}_{to_name}")
    fn.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = None
    return fn


def set_wide(wide: bool):
    load().oracle_set_wide(1 if wide else 0)


def set_reduce_parallel(on: bool):
    load().oracle_set_reduce_parallel(1 if on else 0)


def set_num_threads(n: int):
    load().oracle_set_num_threads(int(n))


def max_threads() -> int:
    return load().oracle_get_max_threads()
