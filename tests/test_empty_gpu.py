"""Empty tensors (num_els == 0, a zero extent among the dims) through every family of the C ABI: the call is a
no-op - no launch error, no sticky status, nothing written - as a loop over zero elements is in the reference."""
import ctypes

import numpy as np
import pytest

from maidenx_b200 import _lib, device

pytestmark = pytest.mark.gpu
SZ = ctypes.c_size_t


def test_zero_element_calls_are_no_ops(cuda):
    lib = _lib.load()
    guard = np.full(64, 7.0, dtype=np.float32)
    a, b, o = (device.CudaBuffer.from_host(guard) for _ in range(3))
    z = SZ(0)

    def call(op, dt, meta, *args):
        device.dispatch(op, dt, meta, *args)  # raises on a sticky error

    call("add", "f32", [0, 4, 4, 1, 4, 1, 0, 0], z, SZ(2), "META", a.ptr, b.ptr, o.ptr)
    call("add_inplace", "f32", [0, 1, 1, 0, 0], z, SZ(1), "META", a.ptr, b.ptr)
    call("eq", "i32", [0, 1, 1, 0, 0], z, SZ(1), "META", a.ptr, b.ptr, o.ptr)
    call("exp", "f32", [0, 1, 0], z, SZ(1), "META", a.ptr, o.ptr)
    call("mul_scalar", "f32", [0, 1, 0], z, SZ(1), "META", a.ptr, ctypes.c_float(2.0), o.ptr)
    call("sum", "f32", [0, 4, 4, 1, 4, 1, 0], z, SZ(2), SZ(1), "META", a.ptr, o.ptr)
    call("max", "f32", [0, 1, 1, 1, 0], z, SZ(1), SZ(1), "META", a.ptr, o.ptr)
    call("sum_to_shape", "f32", [0, 4, 4, 1, 0, 4, 0], z, SZ(2), "META", a.ptr, o.ptr)
    # folding zero rows into a [1, 4] output is not empty on the output side: the reference zero-fills it
    # (crates/maidenx_cpu/src/ops/reduction.rs:91-183), and so does the library
    s2 = device.CudaBuffer.from_host(guard)
    call("sum_to_shape", "f32", [0, 4, 4, 1, 1, 4, 0], z, SZ(2), "META", a.ptr, s2.ptr)
    assert np.array_equal(s2.to_host(np.float32, 8), np.array([0, 0, 0, 0, 7, 7, 7, 7], dtype=np.float32))
    s2.free()
    call("matmul", "f32", [2, 2, 2, 0, 4, 0, 3, 3, 4, 3, 1, 4, 1, 0, 0], z, "META", a.ptr, b.ptr, o.ptr)
    call("matmul_backward", "f32", [2, 2, 2, 0, 4, 0, 3, 3, 4, 3, 1, 4, 1, 0, 0], z, SZ(12), "META", o.ptr, a.ptr, b.ptr, None, None)
    call("conv2d_im2col", "f32", [0, 3, 8, 8, 3, 3, 8, 8, 1, 1, 1, 1], z, "META", a.ptr, o.ptr)
    call("conv2d_col2im", "f32", [0, 3, 8, 8, 3, 3, 8, 8, 1, 1, 1, 1], z, "META", a.ptr, o.ptr)
    call("fold", "f32", [0, 2, 2, 1, 0, 1, 3, 1, 2, 0], z, SZ(2), "META", a.ptr, o.ptr)
    pad_meta = [0, 1, 0, 3, 1, 2]
    call("pad_with_constant", "f32", pad_meta, z, z, SZ(1), "META", a.ptr, o.ptr, ctypes.c_float(1.0))
    call("pad_with_reflection", "f32", pad_meta, z, z, SZ(1), "META", a.ptr, o.ptr)
    call("pad_with_replication_backward", "f32", pad_meta, z, z, SZ(1), "META", a.ptr, o.ptr)
    call("softmax", "f32", [0, 4, 4, 1, 0], z, SZ(2), SZ(1), "META", a.ptr, o.ptr)
    meta = np.array([0, 1, 0], dtype=np.uint64)
    _lib.contiguous("f32")(z, SZ(1), meta.ctypes.data, a.ptr, o.ptr)
    _lib.cast("f32", "i32")(z, a.ptr, o.ptr)
    lib.mx_bias_gelu_f32(0, a.ptr, b.ptr, o.ptr, None)
    lib.mx_sgd_update_f32(0, a.ptr, b.ptr, o.ptr, ctypes.c_float(0.1), ctypes.c_float(1.0))
    device.synchronize()
    assert device.last_error() is None
    for buf in (a, b, o):
        assert np.array_equal(buf.to_host(np.float32, 64), guard)
        buf.free()
