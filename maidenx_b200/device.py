"""Device memory and the reference-style dispatch pattern, through the library's own wrappers.

`CudaBuffer` mirrors the reference's buffer type (crates/maidenx_core/src/buffer/cuda.rs:21-40,
58-75): `cuda_malloc` on creation, `cuda_free` on release, base pointer handed to the ops,
element offsets travelling in the metadata.  `dispatch` mirrors what every generated
function of crates/maidenx_core/src/be/ops/*.rs does around an op call: select the device,
upload the metadata block with cuda_malloc + cuda_memcpy_h2d, call `cuda_<op>_<dtype>`,
free the block.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib


class CudaError(RuntimeError):
    pass


def _check(code: int, what: str):
    if code != 0:
        lib = _lib.load()
        raise CudaError(f"{what}: {lib.cuda_error_string(code).decode()} ({code})")


class CudaBuffer:
    def __init__(self, nbytes: int):
        lib = _lib.load()
        self.nbytes = int(nbytes)
        p = ctypes.c_void_p()
        _check(lib.cuda_malloc(ctypes.byref(p), max(self.nbytes, 1)), "cuda_malloc")
        self.ptr = p.value

    @classmethod
    def from_host(cls, arr: np.ndarray) -> "CudaBuffer":
        arr = np.ascontiguousarray(arr)
        buf = cls(arr.nbytes)
        if arr.nbytes:
            _check(_lib.load().cuda_memcpy_h2d(buf.ptr, arr.ctypes.data, arr.nbytes), "cuda_memcpy_h2d")
        return buf

    def to_host(self, np_dtype, count: int) -> np.ndarray:
        out = np.empty(count, dtype=np_dtype)
        if out.nbytes:
            _check(_lib.load().cuda_memcpy_d2h(out.ctypes.data, self.ptr, out.nbytes), "cuda_memcpy_d2h")
        return out

    def fill_from(self, arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        _check(_lib.load().cuda_memcpy_h2d(self.ptr, arr.ctypes.data, arr.nbytes), "cuda_memcpy_h2d")

    def free(self):
        if self.ptr:
            _lib.load().cuda_free(self.ptr)
            self.ptr = None

    def __del__(self):  # pragma: no cover
        try:
            self.free()
        except Exception:
            pass


def alloc_and_copy_dims(metadata) -> CudaBuffer:
    """crates/maidenx_cuda/src/lib.rs:177-193."""
    return CudaBuffer.from_host(np.asarray(metadata, dtype=np.uint64))


def last_error() -> str | None:
    lib = _lib.load()
    st = lib.mx_last_error()
    if st == 0:
        return None
    msg = f"status {st} at {lib.mx_last_error_where().decode()}"
    if st == 1:
        msg += f": {lib.cuda_error_string(lib.mx_last_cuda_error()).decode()}"
    return msg


def dispatch(op: str, dtype_name: str, metadata, *args, device: int = 0, metadata_on_host: bool = False, check: bool = True):
    """Call cuda_<op>_<dtype> the way maidenx_core does.  `args` is the op's argument list
    with the string "META" standing where the metadata pointer goes."""
    lib = _lib.load()
    _check(lib.cuda_set_device(device), "cuda_set_device")
    fn = _lib.op(op, dtype_name)
    mbuf = None
    keep = None
    if metadata is None:
        mptr = None
    elif metadata_on_host:
        keep = np.asarray(metadata, dtype=np.uint64)
        mptr = keep.ctypes.data
    else:
        mbuf = alloc_and_copy_dims(metadata)
        mptr = mbuf.ptr
    call_args = [mptr if (isinstance(a, str) and a == "META") else a for a in args]
    fn(*call_args)
    if mbuf is not None:
        mbuf.free()
    if check:
        err = last_error()
        if err:
            lib.mx_clear_error()
            raise CudaError(f"cuda_{op}_{dtype_name}: {err}")


def synchronize():
    _check(_lib.load().mx_device_synchronize(), "cudaDeviceSynchronize")
