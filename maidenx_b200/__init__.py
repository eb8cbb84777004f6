"""Blackwell (sm_100a) implementation of the MaidenX CUDA op layer.

The product is `libmaidenx_cuda.so` (sources under `csrc/`, C ABI in
`include/maidenx_cuda.h`).  The Python modules here are the thin host side used by the
tests and the benchmark: a ctypes loader, dtype tables, device buffers that go through
the library's own `cuda_malloc` / `cuda_memcpy_*` wrappers, and the reference-style
dispatch (`upload metadata -> call -> free`).
"""
from . import dtypes  # noqa: F401
from ._lib import LibraryMissing, load, op  # noqa: F401
