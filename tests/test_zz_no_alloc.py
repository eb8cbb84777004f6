"""mx_sum_f32_noalloc — the reduction for callers that cannot allocate device memory (hot loops
that must stay free of driver allocation calls, processes whose allocator owns the whole GPU) —
must give what cuda_sum_f32 gives, call after call, from its fixed in-library workspace.

This file is named to be collected last, so a run that stops at the first failure has already
executed every other test.  It passes alone in a fresh process and after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest

from maidenx_b200 import _lib, device

pytestmark = pytest.mark.gpu
SZ = ctypes.c_size_t


def _both(lib, x_buf, dims, dim, n_out):
    strides = [int(np.prod(dims[i + 1:])) for i in range(len(dims))]
    meta = np.asarray(list(dims) + strides + [dims[dim], strides[dim], 0], dtype=np.uint64)
    n = int(np.prod(dims))
    out_a, out_b = device.CudaBuffer(n_out * 4), device.CudaBuffer(n_out * 4)
    # dirty outputs: both entry points must overwrite
    junk = np.full(n_out, 123.0, np.float32)
    out_a.fill_from(junk)
    out_b.fill_from(junk)
    _lib.op("sum", "f32")(SZ(n), SZ(len(dims)), SZ(1), meta.ctypes.data, x_buf.ptr, out_a.ptr)
    lib.mx_sum_f32_noalloc(n, len(dims), 1, meta.ctypes.data, x_buf.ptr, out_b.ptr)
    device.synchronize()
    a, b = out_a.to_host(np.float32, n_out), out_b.to_host(np.float32, n_out)
    out_a.free()
    out_b.free()
    return a, b


def test_noalloc_sum_matches_regular_sum_on_repeated_calls():
    lib = _lib.load()
    assert lib.cuda_set_device(0) == 0
    rng = np.random.default_rng(42)
    cases = [([3000, 256], 0, 256),      # column fold, split over blocks: partials in the fixed workspace
             ([6, 70001], 1, 6),          # few long rows, split: partials in the fixed workspace
             ([40, 50, 36], 1, 1440),     # middle fold
             ([123457], 0, 1)]            # full reduction
    for _ in range(2):                    # two calls in a row share (and must not depend on) the workspace
        for dims, dim, n_out in cases:
            x = rng.standard_normal(int(np.prod(dims))).astype(np.float32)
            xb = device.CudaBuffer.from_host(x)
            a, b = _both(lib, xb, dims, dim, n_out)
            xb.free()
            assert device.last_error() is None
            # same kernels, same split, same order: bit-identical, which is tighter than the
            # 1e-4 relative bound the reduction tests hold against the oracle
            assert np.array_equal(a, b), (dims, dim, np.abs(a - b).max())
            ref = x.reshape(dims).astype(np.float64).sum(axis=dim).ravel()
            assert np.allclose(b, ref, rtol=1e-4, atol=1e-4 * np.sqrt(dims[dim]))


def test_noalloc_rejects_reductions_beyond_its_workspace_and_device_metadata():
    lib = _lib.load()
    # scatter path (two reduced dims) with more outputs than the 1 MiB workspace holds (262144 floats)
    dims = [2, 300000, 2]
    n = int(np.prod(dims))
    x = device.CudaBuffer(n * 4)
    out = device.CudaBuffer.from_host(np.full(300000, 5.0, np.float32))
    meta = np.asarray(dims + [600000, 2, 1] + [2, 2] + [600000, 1] + [0], dtype=np.uint64)
    lib.mx_clear_error()
    lib.mx_sum_f32_noalloc(n, 3, 2, meta.ctypes.data, x.ptr, out.ptr)
    device.synchronize()
    assert lib.mx_last_error() == 3
    assert np.all(out.to_host(np.float32, 300000) == 5.0)
    lib.mx_clear_error()
    # metadata must be host memory
    mdev = device.CudaBuffer.from_host(np.asarray([4, 1, 4, 1, 0], dtype=np.uint64))
    lib.mx_sum_f32_noalloc(4, 1, 1, mdev.ptr, x.ptr, out.ptr)
    assert lib.mx_last_error() == 2
    lib.mx_clear_error()
    for b in (x, out, mdev):
        b.free()


def test_noalloc_paths_the_first_test_does_not_reach(oracle):
    """Against the CPU oracle (wide accumulation, 1e-4 of max(|ref|, sqrt(terms))): the scatter path (two reduced
    dims), more rows than a grid has y-blocks, rows shorter than a warp, and an input that starts at element 1."""
    import harness as H
    from maidenx_b200 import dtypes as D
    from oracle import binding
    lib = _lib.load()
    rng = np.random.default_rng(43)
    cases = [
        # dims, strides, reduced lens, reduced strides, offset, terms per output
        ([6, 5, 7], [35, 7, 1], [6, 7], [35, 1], 0, 42),        # two reduced dims: scatter path, workspace zero-filled per call
        ([70000, 40], [40, 1], [40], [1], 0, 40),               # 70000 rows: beyond the grid's y limit
        ([5000, 7], [7, 1], [7], [1], 0, 7),                    # rows shorter than a warp
        ([300, 1000], [1000, 1], [1000], [1], 1, 1000),         # the reference's fixture layout: offset 1, not 16-byte aligned
        ([2000, 96], [96, 1], [2000], [96], 1, 2000),           # column fold at offset 1
    ]
    for _ in range(2):
        for dims, strides, rl, rs, off, terms in cases:
            n = int(np.prod(dims))
            x = rng.standard_normal(n + off).astype(np.float32)
            n_out = n // int(np.prod(rl))
            binding.set_wide(True)
            try:
                ref = H.run_reduce(oracle, "sum", D.F32, dims, strides, rl, rs, off, x)
            finally:
                binding.set_wide(False)
            xb = device.CudaBuffer.from_host(x)
            ob = device.CudaBuffer.from_host(np.full(n_out, 9.0, np.float32))
            meta = np.asarray(dims + strides + rl + rs + [off], dtype=np.uint64)
            lib.mx_sum_f32_noalloc(n, len(dims), len(rl), meta.ctypes.data, xb.ptr, ob.ptr)
            device.synchronize()
            assert device.last_error() is None, (dims, device.last_error())
            got = ob.to_host(np.float32, n_out)
            xb.free()
            ob.free()
            H.assert_same("sum", D.F32, got, ref, float_rel=1e-4, scale=np.sqrt(terms), what=f"noalloc {dims} reduce {rl} offset {off}")
