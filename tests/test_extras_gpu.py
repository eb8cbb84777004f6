"""fold, the three paddings (forward and backward) and softmax on a B200 against the CPU oracle,
through the C ABI.  Bar: paddings forward are copies - bit-exact for every dtype; fold and the
padding backward passes are sums - bit-exact for integers (wrapping), floats against the oracle's
wide mode (f32 accumulation for 16-bit, f64 for f32) within f32 1e-5 / 16-bit 1e-2 of the largest
magnitude involved; softmax within f32 1e-5, f64 1e-12, 16-bit 2e-2.  Layouts: the reference's
golden fixtures (offset 1), larger random shapes, transposed and broadcast inputs."""
import json
from pathlib import Path

import numpy as np
import pytest

import harness as H
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu
GOLD = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())


def _sum_tol(dt):
    return {"f32": 1e-5, "f64": 1e-12, "bf16": 1e-2, "f16": 1e-2}.get(dt.name, 0.0)


def _close(got, ref, dt, scale):
    if dt.kind != "float":
        assert np.array_equal(got, ref), (dt.name, got[:8], ref[:8])
        return
    g, r = D.decode(got, dt).astype(np.float64), D.decode(ref, dt).astype(np.float64)
    assert np.all(np.abs(g - r) <= _sum_tol(dt) * np.maximum(np.abs(r), scale)), (dt.name, np.abs(g - r).max())


PAD_LAYOUTS = [
    # name, in_dims, in_strides, offset, pads
    ("1d", [37], [1], 3, [(4, 9)]),
    ("2d", [19, 33], [33, 1], 0, [(2, 3), (5, 1)]),
    ("2d-transposed", [19, 33], [1, 19], 1, [(1, 0), (0, 7)]),
    ("3d", [5, 12, 21], [252, 21, 1], 0, [(0, 0), (3, 3), (2, 4)]),
    ("3d-no-pad", [4, 6, 8], [48, 8, 1], 2, [(0, 0), (0, 0), (0, 0)]),
    ("4d-image", [2, 3, 17, 23], [3 * 17 * 23, 17 * 23, 23, 1], 0, [(0, 0), (0, 0), (2, 2), (3, 3)]),
    ("4d-image-pad1", [3, 5, 56, 56], [5 * 56 * 56, 56 * 56, 56, 1], 0, [(0, 0), (0, 0), (1, 1), (1, 1)]),
    ("rows-of-vectors", [6, 64], [64, 1], 0, [(1, 2), (8, 8)]),
    ("size-1-dims", [1, 9, 1, 16], [999, 16, 7, 1], 0, [(1, 1), (0, 2), (0, 0), (3, 5)]),
    ("first-dim-only", [11, 40], [40, 1], 4, [(3, 2), (0, 0)]),
    # image batches of 64 planes or more are staged plane-wise through shared memory
    ("image-batch-odd", [4, 40, 17, 23], [40 * 17 * 23, 17 * 23, 23, 1], 0, [(0, 0), (0, 0), (2, 2), (3, 3)]),
    ("image-batch-offset", [2, 50, 24, 24], [50 * 576, 576, 24, 1], 3, [(0, 0), (0, 0), (1, 1), (1, 1)]),
    ("image-batch-one-side", [70, 12, 20], [240, 20, 1], 0, [(0, 0), (0, 5), (4, 0)]),
]


@pytest.mark.parametrize("mode", ["constant", "reflection", "replication"])
def test_padding_forward_and_backward(oracle, cuda, mode):
    rng = np.random.default_rng(len(mode))
    oracle.b.set_wide(True)
    try:
        for dt in D.ARITH:
            for name, dims, strides, off, pads in PAD_LAYOUTS:
                n_in = H.numel(dims)
                span = off + sum((d - 1) * s for d, s in zip(dims, strides)) + 1
                x = H.full_range_store(rng, dt, span) if dt.kind != "float" else H.random_store(rng, dt, span, dist="normal")
                value = 3 if dt.kind != "float" else 1.5
                ref = H.run_pad(oracle, mode, dt, dims, strides, off, pads, x, value)
                got = H.run_pad(cuda, mode, dt, dims, strides, off, pads, x, value)
                assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), (mode, dt.name, name)
                n_out = got.size
                g = H.random_store(rng, dt, n_out, dist="normal") if dt.kind == "float" else H.random_store(rng, dt, n_out, lo=-100, hi=100)
                gref = H.run_pad_backward(oracle, mode, dt, dims, strides, off, pads, g, off + n_in + 3)
                ggot = H.run_pad_backward(cuda, mode, dt, dims, strides, off, pads, g, off + n_in + 3)
                # outside [off, off + n_in) the buffer is untouched (both backends were handed the same dirty buffer)
                _close(ggot, gref, dt, scale=4.0)
    finally:
        oracle.b.set_wide(False)


def test_padding_and_fold_golden_vectors(cuda):
    for rec in GOLD["padding"]:
        for dt in (D.F32, D.F64, D.BF16, D.I32):
            if rec["value"] is not None and rec["value"] != int(rec["value"]) and dt.kind != "float":
                continue
            shape, pads = rec["shape"], [tuple(p) for p in rec["pads"]]
            store = np.concatenate([D.encode([0.0], dt), D.encode(rec["input"], dt)])
            got = H.run_pad(cuda, rec["mode"], dt, shape, H.contiguous_strides(shape), 1, pads, store, rec["value"])
            assert np.allclose(D.decode(got, dt).astype(np.float64), np.array(rec["expected"]), atol=0.1 if dt is D.BF16 else 1e-6), (rec["cite"], dt.name)
            if rec["grad"] is not None:
                gi = H.run_pad_backward(cuda, rec["mode"], dt, shape, H.contiguous_strides(shape), 0, pads, D.encode(np.ones(len(rec["expected"])), dt),
                                        len(rec["input"]))
                assert np.allclose(D.decode(gi, dt).astype(np.float64), np.array(rec["grad"]), atol=0.1 if dt is D.BF16 else 0), (rec["cite"], dt.name)
    for rec in GOLD["fold"]:
        for dt in (D.F32, D.BF16, D.I64, D.U8):
            shape, dim, size, step = rec["shape"], rec["dim"], rec["size"], rec["step"]
            st = H.contiguous_strides(shape)
            nwin = (shape[dim] - size) // step + 1
            dims = shape[:dim] + [nwin, size] + shape[dim + 1:]
            strides = st[:dim] + [step * st[dim], st[dim]] + st[dim + 1:]
            store = np.concatenate([D.encode([0.0], dt), D.encode(rec["input"], dt)])
            got = H.run_fold(cuda, dt, dims, strides, dim, dim + 1, shape[dim], step, 1, store)
            assert np.allclose(D.decode(got, dt).astype(np.float64), np.array(rec["expected"]), atol=0.1 if dt is D.BF16 else 0), (rec["cite"], dt.name)


FOLD_CASES = [
    # name, original shape, dim, window, step
    ("1d-overlap", [1000], 0, 7, 3),
    ("1d-gaps", [1000], 0, 2, 5),
    ("2d-inner", [37, 129], 1, 16, 4),
    ("2d-outer", [64, 50], 0, 8, 8),
    ("3d-middle", [6, 40, 11], 1, 5, 2),
]


def test_fold(oracle, cuda):
    rng = np.random.default_rng(11)
    oracle.b.set_wide(True)
    try:
        for dt in D.ARITH:
            for name, shape, dim, size, step in FOLD_CASES:
                st = H.contiguous_strides(shape)
                nwin = (shape[dim] - size) // step + 1
                # (a) the view unfold() makes of a dense tensor: windows overlap in memory
                dims = shape[:dim] + [nwin, size] + shape[dim + 1:]
                strides = st[:dim] + [step * st[dim], st[dim]] + st[dim + 1:]
                x = H.random_store(rng, dt, H.numel(shape) + 2, dist="normal") if dt.kind == "float" else H.random_store(rng, dt, H.numel(shape) + 2, lo=-50, hi=50)
                fold_size = (nwin - 1) * step + size
                ref = H.run_fold(oracle, dt, dims, strides, dim, dim + 1, fold_size, step, 2, x)
                got = H.run_fold(cuda, dt, dims, strides, dim, dim + 1, fold_size, step, 2, x)
                _close(got, ref, dt, scale=4.0)
                # (b) a dense gradient of the unfolded shape (what backward hands over)
                g = H.random_store(rng, dt, H.numel(dims), dist="normal") if dt.kind == "float" else H.random_store(rng, dt, H.numel(dims), lo=-50, hi=50)
                ref = H.run_fold(oracle, dt, dims, H.contiguous_strides(dims), dim, dim + 1, fold_size, step, 0, g)
                got = H.run_fold(cuda, dt, dims, H.contiguous_strides(dims), dim, dim + 1, fold_size, step, 0, g)
                _close(got, ref, dt, scale=4.0)
    finally:
        oracle.b.set_wide(False)


SOFTMAX_CASES = [
    ("rows", [64, 1000], [1000, 1], 0, 1),
    ("cols", [300, 48], [48, 1], 0, 0),
    ("middle", [7, 129, 5], [645, 5, 1], 1, 1),
    ("last-by-default", [9, 33], [33, 1], 0, 5),
    ("transposed", [40, 24], [1, 40], 0, 1),
    ("long", [3, 20000], [20000, 1], 0, 1),
    # rows held in registers: one warp per row (up to 8 vectors per lane), one block per row beyond that
    ("warp-rows", [70, 256], [256, 1], 0, 1),
    ("warp-rows-partial", [33, 1000], [1000, 1], 8, 1),
    ("block-rows", [5, 4096], [4096, 1], 0, 1),
    ("block-rows-ragged", [3, 8200], [8200, 1], 0, 1),
    ("block-rows-max", [2, 16384], [16384, 1], 0, 1),
    ("rows-unaligned-offset", [6, 512], [512, 1], 3, 1),      # not 16-byte aligned: general kernel
    ("cols-wide", [3, 50, 64], [3200, 64, 1], 0, 1),          # one thread per column
    ("cols-first-dim", [200, 160], [160, 1], 0, 0),
    ("cols-odd-extent", [9, 40, 18], [720, 18, 1], 0, 1),     # trailing extent not a multiple of the vector: one column per lane
]


def test_softmax(oracle, cuda):
    rng = np.random.default_rng(12)
    oracle.b.set_wide(True)
    try:
        for dt in D.FLOATS:
            for name, dims, strides, off, dim in SOFTMAX_CASES:
                span = off + sum((d - 1) * s for d, s in zip(dims, strides)) + 1
                x = D.encode(rng.standard_normal(span) * 3.0, dt)
                ref = D.decode(H.run_softmax(oracle, dt, dims, strides, off, dim, x), dt).astype(np.float64)
                got = D.decode(H.run_softmax(cuda, dt, dims, strides, off, dim, x), dt).astype(np.float64)
                tol = {"f32": 1e-5, "f64": 1e-12, "bf16": 2e-2, "f16": 2e-2}[dt.name]
                assert np.all(np.abs(got - ref) <= tol * np.maximum(np.abs(ref), 1e-30 if dt.name in ("f32", "f64") else 1e-4)), (dt.name, name, np.abs(got - ref).max())
                axis = dim if dim < len(dims) else len(dims) - 1
                assert np.allclose(got.reshape(dims).sum(axis=axis), 1.0, atol=2e-2 if dt.name in ("bf16", "f16") else 1e-5)
    finally:
        oracle.b.set_wide(False)


CONTIGUOUS_VIEWS = [
    # name, dims, strides, offset
    ("dense", [33, 65], [65, 1], 0),
    ("transposed", [128, 192], [1, 128], 0),
    ("transposed-odd", [67, 131], [1, 67], 3),
    ("permuted-3d", [5, 6, 7], [1, 35, 5], 0),
    ("broadcast-rows", [40, 72], [0, 1], 2),
    ("sliced-rows", [30, 50], [120, 2], 1),
    ("batched-transpose", [3, 40, 72], [2880, 1, 40], 0),
    ("scalar", [], [], 4),
]


def test_contiguous_copies_any_view_bit_exact(cuda):
    """mx_contiguous_<T> against numpy's strided gather, every dtype: the device-side Tensor::contiguous()."""
    import ctypes

    from maidenx_b200 import _lib, device
    rng = np.random.default_rng(21)
    for dt in D.ALL:
        fn = _lib.contiguous(dt.name)
        for name, dims, strides, off in CONTIGUOUS_VIEWS:
            span = off + sum((d - 1) * s for d, s in zip(dims, strides)) + 1
            x = H.full_range_store(rng, dt, span + 5)
            n = H.numel(dims)
            want = np.lib.stride_tricks.as_strided(x[off:], shape=dims, strides=[s * x.itemsize for s in strides]).reshape(-1) if dims else x[off:off + 1]
            xb, ob = device.CudaBuffer.from_host(x), device.CudaBuffer.from_host(np.full(max(n, 1), 7).astype(dt.np_storage))
            meta = np.asarray(list(dims) + list(strides) + [off], dtype=np.uint64)
            fn(ctypes.c_size_t(n), ctypes.c_size_t(len(dims)), meta.ctypes.data, xb.ptr, ob.ptr)
            device.synchronize()
            got = ob.to_host(dt.np_storage, n)
            assert device.last_error() is None
            assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8)), (dt.name, name)
            xb.free()
            ob.free()


def _cast_inputs(rng, dt, n):
    """Values that exercise every rule: the whole integer range, fractions, huge magnitudes, NaN and infinities."""
    if dt.kind == "float":
        v = rng.standard_normal(n) * 10.0 ** rng.integers(-3, 12, n)
        v[: min(n, 12)] = [0.0, -0.0, 1.5, -1.5, 255.5, -129.2, 65536.7, 3e9, -3e9, np.nan, np.inf, -np.inf][: min(n, 12)]
        return D.encode(v if dt is D.F64 else v.astype(np.float32), dt)
    return H.full_range_store(rng, dt, n)


def test_casts_match_the_oracle_bit_for_bit(cuda):
    """All 169 ordered dtype pairs of mx_cast_<from>_<to> against the oracle's element rules, on an odd length
    (vector body + scalar tail) and from a misaligned base (scalar path)."""
    import ctypes

    from maidenx_b200 import _lib, device
    from oracle import binding
    rng = np.random.default_rng(33)
    n = 4099
    for sdt in D.ALL:
        x = _cast_inputs(rng, sdt, n + 3)
        xb = device.CudaBuffer.from_host(x)
        for ddt in D.ALL:
            for shift in (0, 3):  # element offset of the views handed to the op
                src = x[shift:shift + n - shift]
                m = src.size
                want = np.zeros(m, dtype=ddt.np_storage)
                binding.cast(sdt.name, ddt.name)(m, np.ascontiguousarray(src).ctypes.data, want.ctypes.data)
                ob = device.CudaBuffer.from_host(np.full(m + 8, 7).astype(ddt.np_storage))
                _lib.cast(sdt.name, ddt.name)(ctypes.c_size_t(m), xb.ptr + shift * sdt.size, ob.ptr + shift * ddt.size)
                device.synchronize()
                assert device.last_error() is None
                got = ob.to_host(ddt.np_storage, m + 8)[shift:shift + m]
                if ddt.kind == "float":  # NaNs may differ in payload between the CPU and GPU conversions: compare as a class
                    g, w = D.decode(got, ddt), D.decode(want, ddt)
                    assert np.array_equal(np.isnan(g), np.isnan(w)), (sdt.name, ddt.name)
                    ok = ~np.isnan(w)
                    assert np.array_equal(got[ok].view(np.uint8), want[ok].view(np.uint8)), (sdt.name, ddt.name, shift)
                else:
                    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (sdt.name, ddt.name, shift)
                ob.free()
        xb.free()


def test_softmax_special_values(oracle, cuda):
    """-inf terms (alone in a slice, beside finite values, as a slice's first or last element), +inf and NaN: the row
    kernel, the column kernel (which folds the maximum and the sum into one pass) and the general kernel must place NaN
    and zeros where the reference's three-pass form does."""
    rng = np.random.default_rng(99)
    oracle.b.set_wide(True)
    try:
        for dt in (D.F32, D.BF16):
            for dims, dim in (([12, 256], 1), ([300, 64], 0), ([5, 40, 18], 1), ([7, 33], 1)):
                n = int(np.prod(dims))
                x = rng.standard_normal(n) * 3.0
                v = x.reshape(dims)
                sl = [slice(None)] * len(dims)

                def at(i, j):  # slice i along the softmax dim, position j inside it
                    idx = [0] * len(dims)
                    idx[dim] = j
                    other = [d for d in range(len(dims)) if d != dim]
                    rem = i
                    for d in reversed(other):
                        idx[d] = rem % dims[d]
                        rem //= dims[d]
                    return tuple(idx)

                L = dims[dim]
                v[at(0, 0)] = -np.inf                      # first element of a slice
                v[at(1, L - 1)] = -np.inf                  # last element
                for j in range(L):
                    v[at(2, j)] = -np.inf                  # a slice of nothing but -inf
                v[at(3, L // 2)] = np.inf                  # one +inf
                v[at(4, 1)] = np.nan                       # one NaN
                v[at(5, 0)] = -np.inf
                v[at(5, 3)] = np.nan                       # -inf first, NaN later
                xs = D.encode(v.reshape(-1), dt)
                strides = H.contiguous_strides(dims)
                ref = D.decode(H.run_softmax(oracle, dt, dims, strides, 0, dim, xs), dt).astype(np.float64)
                got = D.decode(H.run_softmax(cuda, dt, dims, strides, 0, dim, xs), dt).astype(np.float64)
                assert np.array_equal(np.isnan(got), np.isnan(ref)), (dt.name, dims, dim)
                ok = ~np.isnan(ref)
                tol = 1e-5 if dt.name == "f32" else 2e-2
                assert np.all(np.abs(got[ok] - ref[ok]) <= tol * np.maximum(np.abs(ref[ok]), 1e-30 if dt.name == "f32" else 1e-4)), (dt.name, dims, dim)
    finally:
        oracle.b.set_wide(False)
