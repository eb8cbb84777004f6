"""Parity of sum / mean / max / min and sum_to_shape against the CPU oracle, through the
C ABI, on a B200.

Bar: integers bit-exact (wrapping sums are order-independent); max / min bit-exact for
every dtype (the result is one of the inputs); float sums and means against the oracle's
wide-accumulator evaluation of the same formulas: f32 within 1e-4, f64 1e-12, bf16 / f16
2e-2, each relative to max(|ref|, sqrt(R) * sigma) where R is the number of folded terms
(the natural scale of a sum of R zero-mean terms).  Output buffers are handed over dirty
(the ops must overwrite), and every case is run twice to check bitwise determinism.
Shapes are chosen to hit every kernel: thread / warp / block rows, split rows, vector and
scalar column strips, split columns, the [O,R,I] middle fold, and the literal scatter
path (several reduced dims, non-contiguous input, broadcast input, partial factors).
"""
import numpy as np
import pytest

import harness as H
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu

SUM_TOL = {"f32": 1e-4, "f64": 1e-12, "bf16": 2e-2, "f16": 2e-2}


def dim_cases():
    """(name, dims, strides or None for contiguous, reduced dims, offset)"""
    return [
        ("rows-thread", [300, 7], None, [1], 0),
        ("rows-warp", [2000, 96], None, [1], 0),
        ("rows-warp-odd", [777, 101], None, [1], 0),
        ("rows-block", [40, 5000], None, [1], 0),
        ("rows-block-vec", [24, 4096], None, [1], 0),
        ("rows-split", [3, 70001], None, [1], 0),
        ("sum-all", [123457], None, [0], 0),
        ("cols-vec", [500, 256], None, [0], 0),
        ("cols-odd", [333, 77], None, [0], 0),
        ("cols-split", [4000, 64], None, [0], 0),
        ("cols-narrow", [900, 3], None, [0], 0),
        ("middle", [6, 50, 40], None, [1], 0),
        ("middle-narrow", [5, 33, 2], None, [1], 0),
        ("offset1", [64, 33], None, [0], 1),
        ("offset1-rows", [33, 64], None, [1], 1),
        ("len1", [17, 1, 9], None, [1], 0),
        ("two-dims", [6, 7, 8], None, [0, 2], 0),
        ("transposed-input", [12, 10], [1, 12], [0], 0),
        ("broadcast-input", [4, 6], [0, 1], [0], 0),
    ]


def _run_dim(be, op, dt, dims, strides, red, off, store):
    st = strides or H.contiguous_strides(dims)
    return H.run_reduce(be, op, dt, dims, st, [dims[d] for d in red], [st[d] for d in red], off, store)


def _buffer_len(dims, strides, off):
    if strides is None:
        return H.numel(dims) + off
    return sum((d - 1) * s for d, s in zip(dims, strides)) + 1 + off


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min"])
def test_dim_reductions(oracle, cuda, op):
    from oracle import binding
    rng = np.random.default_rng({"sum": 1, "mean": 2, "max": 3, "min": 4}[op])
    for dt in (D.FLOATS if op == "mean" else D.ARITH):
        for name, dims, strides, red, off in dim_cases():
            blen = _buffer_len(dims, strides, off)
            if op in ("max", "min"):
                store = H.full_range_store(rng, dt, blen)
            elif dt.kind == "float":
                store = H.random_store(rng, dt, blen, dist="normal")
            else:
                store = H.full_range_store(rng, dt, blen)  # wrapping sums
            binding.set_wide(op in ("sum", "mean") and dt.kind == "float")
            try:
                ref = _run_dim(oracle, op, dt, dims, strides, red, off, store)
            finally:
                binding.set_wide(False)
            got = _run_dim(cuda, op, dt, dims, strides, red, off, store)
            again = _run_dim(cuda, op, dt, dims, strides, red, off, store)
            assert got.tobytes() == again.tobytes() or (dt.kind == "float" and name in ("two-dims", "transposed-input", "broadcast-input")), \
                f"{name} {op}_{dt.name}: not deterministic"
            if op in ("max", "min") or dt.kind != "float":
                H.assert_same(op, dt, got, ref, what=name)
            else:
                folded = 1
                for d in red:
                    folded *= dims[d]
                scale = np.sqrt(folded) * (1.0 if op == "sum" else 1.0 / folded)
                H.assert_same(op, dt, got, ref, float_rel=SUM_TOL[dt.name], what=name, scale=scale)


def shape_cases():
    """(name, in_dims, strides or None, out_dims, offset)"""
    return [
        ("lead-fold", [64, 96], None, [1, 96], 0),                 # [R, K]
        ("lead-fold-3d", [8, 16, 40], None, [1, 1, 40], 0),        # merged [R, K]
        ("trail-fold", [50, 333], None, [50, 1], 0),               # [K, R]
        ("full-fold", [9, 11, 13], None, [1, 1, 1], 0),            # [R]
        ("middle-fold", [7, 30, 24], None, [7, 1, 24], 0),         # [K, R, K]
        ("bias-fold", [4, 6, 5, 5], None, [1, 6, 1, 1], 0),        # [R, K, R]: literal scatter
        ("no-fold", [5, 8], None, [5, 8], 1),
        ("partial", [4, 6], None, [2, 3], 0),                      # block fold by 2 x 2
        ("offset1", [2, 3], None, [1, 3], 1),
        ("transposed-input", [6, 4], [1, 6], [1, 4], 0),
    ]


def test_sum_to_shape(oracle, cuda):
    from oracle import binding
    rng = np.random.default_rng(11)
    for dt in D.ARITH:
        for name, dims, strides, odims, off in shape_cases():
            blen = _buffer_len(dims, strides, off)
            store = H.random_store(rng, dt, blen, dist="normal") if dt.kind == "float" else H.full_range_store(rng, dt, blen)
            st = strides or H.contiguous_strides(dims)
            binding.set_wide(dt.kind == "float")
            try:
                ref = H.run_sum_to_shape(oracle, dt, dims, st, odims, off, store)
            finally:
                binding.set_wide(False)
            got = H.run_sum_to_shape(cuda, dt, dims, st, odims, off, store)
            if dt.kind != "float":
                H.assert_same("sum_to_shape", dt, got, ref, what=name)
            else:
                folded = H.numel(dims) // H.numel(odims)
                H.assert_same("sum_to_shape", dt, got, ref, float_rel=SUM_TOL[dt.name], what=name, scale=np.sqrt(folded))


def test_f32_max_of_only_negative_infinity_is_type_min(oracle, cuda):
    """max starts from f32::MIN, not -inf (crates/maidenx_cpu/src/ops/reduction.rs:605), and NaNs never win."""
    x = np.array([-np.inf, np.nan, -np.inf, -np.inf, np.nan, -np.inf], dtype=np.float32)
    ref = H.run_reduce(oracle, "max", D.F32, [2, 3], [3, 1], [3], [1], 0, x)
    got = H.run_reduce(cuda, "max", D.F32, [2, 3], [3, 1], [3], [1], 0, x)
    assert np.array_equal(ref, got) and got[0] == np.finfo(np.float32).min
