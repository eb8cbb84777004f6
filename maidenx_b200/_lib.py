"""Loader of libmaidenx_cuda.so.  There is no fallback: without the built CUDA library
every op call fails with an error that says how to build it."""
from __future__ import annotations

import ctypes
from pathlib import Path

from . import _signatures as sig

LIB_PATH = Path(__file__).resolve().parent / "libmaidenx_cuda.so"

_lib = None
_ops = None

RUNTIME_SIGNATURES = {
    "cuda_malloc": ([ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t], ctypes.c_int),
    "cuda_free": ([ctypes.c_void_p], ctypes.c_int),
    "cuda_memcpy_h2d": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t], ctypes.c_int),
    "cuda_memcpy_d2h": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t], ctypes.c_int),
    "cuda_memcpy_d2d": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t], ctypes.c_int),
    "cuda_set_device": ([ctypes.c_int], ctypes.c_int),
    "cuda_get_device": ([ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
    "cuda_stream_create": ([ctypes.POINTER(ctypes.c_void_p)], ctypes.c_int),
    "cuda_stream_destroy": ([ctypes.c_void_p], ctypes.c_int),
    "cuda_stream_synchronize": ([ctypes.c_void_p], ctypes.c_int),
    "cuda_pointer_get_attributes": ([ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int),
    "cuda_error_string": ([ctypes.c_int], ctypes.c_char_p),
    "mx_set_stream": ([ctypes.c_void_p], None),
    "mx_get_stream": ([], ctypes.c_void_p),
    "mx_last_error": ([], ctypes.c_int),
    "mx_last_cuda_error": ([], ctypes.c_int),
    "mx_last_error_where": ([], ctypes.c_char_p),
    "mx_clear_error": ([], None),
    "mx_device_synchronize": ([], ctypes.c_int),
    "mx_metadata_table_size": ([], ctypes.c_int),
    "mx_tc_gemm_status": ([], ctypes.c_int),
    "mx_sum_f32_noalloc": ([ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p], None),
    "mx_mlp_create": ([ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_uint64], ctypes.c_void_p),
    "mx_mlp_destroy": ([ctypes.c_void_p], None),
    "mx_mlp_forward": ([ctypes.c_void_p, ctypes.c_void_p], None),
    "mx_mlp_loss_backward": ([ctypes.c_void_p, ctypes.c_void_p], None),
    "mx_mlp_backward_layer": ([ctypes.c_void_p, ctypes.c_int], None),
    "mx_mlp_sgd_layer": ([ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_float], None),
    "mx_mlp_train_step": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_float], None),
    "mx_mlp_weight_grad": ([ctypes.c_void_p, ctypes.c_int], ctypes.c_void_p),
    "mx_mlp_bias_grad": ([ctypes.c_void_p, ctypes.c_int], ctypes.c_void_p),
    "mx_mlp_master_weight": ([ctypes.c_void_p, ctypes.c_int], ctypes.c_void_p),
    "mx_mlp_master_bias": ([ctypes.c_void_p, ctypes.c_int], ctypes.c_void_p),
    "mx_mlp_weight": ([ctypes.c_void_p, ctypes.c_int], ctypes.c_void_p),
    "mx_mlp_output": ([ctypes.c_void_p], ctypes.c_void_p),
    "mx_mlp_loss_ptr": ([ctypes.c_void_p], ctypes.c_void_p),
    "mx_mlp_loss": ([ctypes.c_void_p], ctypes.c_float),
    "mx_dp_barrier": ([ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p], None),
    "mx_dp_reduce_sgd": ([ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t,
                          ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_int, ctypes.c_void_p], None),
    "mx_mlp_dp_arena_bytes": ([ctypes.c_int, ctypes.c_size_t], ctypes.c_size_t),
    "mx_mlp_create_dp": ([ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_uint64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                          ctypes.c_void_p], ctypes.c_void_p),
    "mx_mlp_train_step_dp": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_float], None),
    "mx_mlp_dp_status": ([ctypes.c_void_p], ctypes.c_uint32),
    "mx_mlp_dp_join": ([ctypes.c_void_p], None),
    "mx_mlp_dp_set_exchange": ([ctypes.c_void_p, ctypes.c_int, ctypes.c_int], ctypes.c_int),
    "mx_set_gemm_sm_limit": ([ctypes.c_int], None),
    "mx_set_gemm_cta_group": ([ctypes.c_int], None),
    "mx_set_small_pool": ([ctypes.c_int], None),
    "mx_debug_elementwise_plan": ([ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                   ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
    "mx_debug_matmul_forward_path": ([ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t),
                                      ctypes.POINTER(ctypes.c_size_t)], ctypes.c_int),
    "mx_debug_matmul_forward_path_f32": ([ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                          ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t),
                                          ctypes.POINTER(ctypes.c_size_t)], ctypes.c_int),
    "mx_debug_tc_gemm_poke_status": ([ctypes.c_int], ctypes.c_int),
    "mx_debug_set_gemm_group_m": ([ctypes.c_int], None),
    "mx_debug_gemm_max_resident_pairs": ([], ctypes.c_int),
    "mx_debug_set_gemm_keep_b": ([ctypes.c_int], None),
    "mx_debug_gemm_keep_b_ctas": ([ctypes.c_int] * 5, ctypes.c_int),
    "mx_debug_splitk_slices": ([ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int], ctypes.c_int),
    "mx_debug_reduce_plan": ([ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_size_t),
                              ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)], ctypes.c_int),
}


class MxConv2d(ctypes.Structure):
    """MxConv2d of include/maidenx_cuda.h."""
    _fields_ = [(n, ctypes.c_size_t) for n in ("batch", "in_channels", "height", "width", "out_channels", "kernel_h", "kernel_w", "stride_h",
                                              "stride_w", "pad_h", "pad_w")]


class LibraryMissing(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    global _lib, _ops
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise LibraryMissing(
            f"{LIB_PATH} is not built; run `python -m maidenx_b200.build` (needs nvcc). "
            "The op layer has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (args, res) in RUNTIME_SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
    P, S, F = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float
    for t in ("bf16", "f16"):
        fn = getattr(lib, f"mx_linear_bias_gelu_{t}")
        fn.argtypes, fn.restype = [S, S, S, P, P, P, P, P], None
    for t in ("bf16", "f16", "f32"):
        for name, args in (("mx_bias_gelu", [S, P, P, P, P]), ("mx_gelu_backward", [S, P, P, P]),
                           ("mx_mse_loss_grad", [S, P, P, P, P]), ("mx_sgd_update", [S, P, P, P, F, F])):
            fn = getattr(lib, f"{name}_{t}")
            fn.argtypes = args
            fn.restype = None
    _ops = sig.bind(lib, "cuda_")
    _lib = lib
    return lib


def cast(from_name: str, to_name: str):
    """`mx_cast_<from>_<to>(num_els, in, out)`: dense dtype conversion on the device."""
    fn = getattr(load(), f"mx_cast_{from_name}_{to_name}")
    fn.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = None
    return fn


def conv2d(dtype_name: str):
    """(mx_conv2d_forward_<dtype>, mx_conv2d_backward_<dtype>): the Conv2d layer composed from the op entry points."""
    lib = load()
    P, C = ctypes.c_void_p, ctypes.POINTER(MxConv2d)
    fwd, bwd = getattr(lib, f"mx_conv2d_forward_{dtype_name}"), getattr(lib, f"mx_conv2d_backward_{dtype_name}")
    fwd.argtypes, fwd.restype = [C, ctypes.c_int, P, P, P, P, P, P], None
    bwd.argtypes, bwd.restype = [C, ctypes.c_int, P, P, P, P, P, P, P], None
    for name in ("mx_conv2d_cols_elems", "mx_conv2d_output_elems"):
        getattr(lib, name).argtypes, getattr(lib, name).restype = [C], ctypes.c_size_t
    lib.mx_conv2d_workspace_elems.argtypes, lib.mx_conv2d_workspace_elems.restype = [C, ctypes.c_int, ctypes.c_int], ctypes.c_size_t
    return fwd, bwd


def contiguous(dtype_name: str):
    """`mx_contiguous_<dtype>(num_els, num_dims, metadata, in, out)`: strided view -> dense copy on the device."""
    fn = getattr(load(), f"mx_contiguous_{dtype_name}")
    fn.argtypes = [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = None
    return fn


def op(name: str, dtype_name: str):
    """The `cuda_<name>_<dtype>` entry point."""
    load()
    try:
        return _ops[(name, dtype_name)]
    except KeyError:
        raise KeyError(f"cuda_{name}_{dtype_name} is not part of the op layer") from None
