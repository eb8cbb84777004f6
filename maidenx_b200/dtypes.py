"""Element types of the op layer and their host representations.

The 13 dtypes are those of the reference (crates/maidenx_core/src/dtype.rs:23-38).
numpy has no bfloat16, so bf16 tensors live on the host as uint16 bit patterns; f16 uses
numpy.float16 (IEEE binary16, same bits as the reference's half::f16).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class DType:
    name: str          # suffix used in the C symbols: cuda_add_<name>
    np_storage: type   # numpy dtype of the stored bits
    size: int          # bytes per element
    kind: str          # "float" | "uint" | "sint" | "bool"
    c_arg: type        # ctypes type of a by-value scalar argument

    def __repr__(self) -> str:  # pragma: no cover
        return f"DType({self.name})"


BF16 = DType("bf16", np.uint16, 2, "float", ctypes.c_uint16)
F16 = DType("f16", np.float16, 2, "float", ctypes.c_uint16)
F32 = DType("f32", np.float32, 4, "float", ctypes.c_float)
F64 = DType("f64", np.float64, 8, "float", ctypes.c_double)
BOOL = DType("bool", np.bool_, 1, "bool", ctypes.c_bool)
U8 = DType("u8", np.uint8, 1, "uint", ctypes.c_uint8)
U16 = DType("u16", np.uint16, 2, "uint", ctypes.c_uint16)
U32 = DType("u32", np.uint32, 4, "uint", ctypes.c_uint32)
U64 = DType("u64", np.uint64, 8, "uint", ctypes.c_uint64)
I8 = DType("i8", np.int8, 1, "sint", ctypes.c_int8)
I16 = DType("i16", np.int16, 2, "sint", ctypes.c_int16)
I32 = DType("i32", np.int32, 4, "sint", ctypes.c_int32)
I64 = DType("i64", np.int64, 8, "sint", ctypes.c_int64)

ALL = [BF16, F16, F32, F64, BOOL, U8, U16, U32, U64, I8, I16, I32, I64]
BY_NAME = {d.name: d for d in ALL}
FLOATS = [BF16, F16, F32, F64]
ARITH = [d for d in ALL if d is not BOOL]
SIGNED = FLOATS + [I8, I16, I32, I64]
INTS = [U8, U16, U32, U64, I8, I16, I32, I64]


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (NaN stays NaN)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    rounded = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    quiet = ((u >> 16) | np.uint32(0x40)).astype(np.uint16)
    return np.where(nan, quiet, rounded)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def encode(values, dt: DType) -> np.ndarray:
    """Host array of real values -> stored representation of dtype `dt`."""
    a = np.asarray(values)
    if dt is BF16:
        return f32_to_bf16_bits(a.astype(np.float32))
    if dt is BOOL:
        return a.astype(np.bool_)
    with np.errstate(over="ignore", invalid="ignore"):
        return a.astype(dt.np_storage)


def decode(stored: np.ndarray, dt: DType) -> np.ndarray:
    """Stored representation -> float64 / int64-ish values convenient for comparison."""
    if dt is BF16:
        return bf16_bits_to_f32(stored).astype(np.float64)
    if dt.kind == "float":
        return stored.astype(np.float64)
    return stored


def scalar_arg(value, dt: DType):
    """ctypes by-value argument for a scalar constant of dtype `dt`."""
    if dt is BF16:
        return ctypes.c_uint16(int(f32_to_bf16_bits(np.array([value], dtype=np.float32))[0]))
    if dt is F16:
        return ctypes.c_uint16(int(np.array([value], dtype=np.float16).view(np.uint16)[0]))
    if dt is BOOL:
        return ctypes.c_bool(bool(value))
    if dt.kind == "float":
        return dt.c_arg(float(value))
    return dt.c_arg(int(value))
