"""ctypes signatures of the op entry points, by family.

The same table serves the CUDA library (`cuda_<op>_<dtype>`, include/maidenx_cuda.h) and
the CPU oracle (`<op>_<dtype>`), whose argument lists are identical.
"""
from __future__ import annotations

import ctypes

from . import dtypes as dt

SZ = ctypes.c_size_t
PTR = ctypes.c_void_p

BINARY_ARITH = ["add", "sub", "mul", "div", "maximum", "minimum"]
BINARY_BOOL = ["logical_and", "logical_or", "logical_xor", "eq", "ne", "lt", "le", "gt", "ge"]
BINARY_INPLACE = ["add_inplace", "sub_inplace", "mul_inplace", "div_inplace"]
UNARY_FLOAT = ["relu", "sigmoid", "tanh", "gelu", "sin", "cos", "tan", "ln", "log10", "log2", "exp", "exp10", "exp2",
               "softplus", "recip"]
UNARY_SIGNED = ["neg", "abs"]
UNARY_ARITH = ["sign", "square", "sqrt"]
UNARY_BOOL = ["logical_not"]
UNARY_CONST_ARITH = ["add_scalar", "sub_scalar", "mul_scalar", "div_scalar", "maximum_scalar", "minimum_scalar", "pow"]
UNARY_CONST_FLOAT = ["leaky_relu", "elu"]
UNARY_CONST_BOOL = ["eq_scalar", "ne_scalar", "lt_scalar", "le_scalar", "gt_scalar", "ge_scalar"]
REDUCE_ARITH = ["sum", "max", "min"]
REDUCE_FLOAT = ["mean"]
PAD_FORWARD = ["pad_with_reflection", "pad_with_replication"]
PAD_BACKWARD = ["pad_with_constant_backward", "pad_with_reflection_backward", "pad_with_replication_backward"]


def op_table():
    """Yield (op, dtype, family) for every op entry point the dispatch layer of the
    reference uses (crates/maidenx_core/src/be/ops/{binary,unary,reduction,matmul}.rs,
    be/nn/conv.rs, be/ops/padding.rs, be/nn/activation.rs)."""
    for d in dt.ARITH:
        for op in BINARY_ARITH:
            yield op, d, "binary"
        for op in BINARY_INPLACE:
            yield op, d, "binary_inplace"
        for op in UNARY_ARITH:
            yield op, d, "unary"
        for op in UNARY_CONST_ARITH:
            yield op, d, "unary_const"
        for op in REDUCE_ARITH:
            yield op, d, "reduce"
        yield "sum_to_shape", d, "sum_to_shape"
        yield "fold", d, "sum_to_shape"
        yield "pad_with_constant", d, "pad_const"
        for op in PAD_FORWARD + PAD_BACKWARD:
            yield op, d, "pad"
        yield "matmul", d, "matmul"
        yield "matmul_backward", d, "matmul_backward"
    for d in dt.ALL:
        for op in BINARY_BOOL:
            yield op, d, "binary_bool"
        for op in UNARY_BOOL:
            yield op, d, "unary_bool"
        for op in UNARY_CONST_BOOL:
            yield op, d, "unary_const_bool"
    for d in dt.SIGNED:
        for op in UNARY_SIGNED:
            yield op, d, "unary"
    for d in dt.FLOATS:
        for op in UNARY_FLOAT:
            yield op, d, "unary"
        for op in UNARY_CONST_FLOAT:
            yield op, d, "unary_const"
        for op in REDUCE_FLOAT:
            yield op, d, "reduce"
        yield "conv2d_im2col", d, "conv"
        yield "conv2d_col2im", d, "conv"
        yield "softmax", d, "softmax"


def argtypes(family: str, d: dt.DType):
    if family in ("binary", "binary_bool"):
        return [SZ, SZ, PTR, PTR, PTR, PTR]
    if family == "binary_inplace":
        return [SZ, SZ, PTR, PTR, PTR]
    if family in ("unary", "unary_bool"):
        return [SZ, SZ, PTR, PTR, PTR]
    if family in ("unary_const", "unary_const_bool"):
        return [SZ, SZ, PTR, PTR, d.c_arg, PTR]
    if family == "reduce":
        return [SZ, SZ, SZ, PTR, PTR, PTR]
    if family == "sum_to_shape":
        return [SZ, SZ, PTR, PTR, PTR]
    if family == "pad":         # (num_els_in, num_els_out, num_dims, metadata, in | grad_out, out | grad_in)
        return [SZ, SZ, SZ, PTR, PTR, PTR]
    if family == "pad_const":   # ... plus the pad value
        return [SZ, SZ, SZ, PTR, PTR, PTR, d.c_arg]
    if family == "softmax":     # (num_els, num_dims, dim, metadata, in, out)
        return [SZ, SZ, SZ, PTR, PTR, PTR]
    if family == "matmul":
        return [SZ, PTR, PTR, PTR, PTR]
    if family == "matmul_backward":
        return [SZ, SZ, PTR, PTR, PTR, PTR, PTR, PTR]
    if family == "conv":
        return [SZ, PTR, PTR, PTR]
    raise KeyError(family)


class Binder:
    """Resolves `<prefix><op>_<dtype>` on first use and sets its ctypes signature.  A symbol
    that is not part of the op layer raises KeyError; one that the library fails to export
    raises AttributeError at the call site."""

    def __init__(self, cdll: ctypes.CDLL, prefix: str):
        self.cdll = cdll
        self.prefix = prefix
        self.family = {(op, d.name): (family, d) for op, d, family in op_table()}
        self.cache = {}

    def __getitem__(self, key):
        fn = self.cache.get(key)
        if fn is None:
            family, d = self.family[key]
            fn = getattr(self.cdll, f"{self.prefix}{key[0]}_{key[1]}")
            fn.argtypes = argtypes(family, d)
            fn.restype = None
            self.cache[key] = fn
        return fn


def bind(cdll: ctypes.CDLL, prefix: str) -> Binder:
    return Binder(cdll, prefix)
