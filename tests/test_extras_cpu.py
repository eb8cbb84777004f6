"""CPU-only checks of the oracle's softmax (the reference pins it by properties only:
crates/maidenx_nn/src/layers/activation/softmax.rs:115-230 - shape, rows summing to one, ordering)."""
import numpy as np
import pytest

import harness as H
from maidenx_b200 import dtypes as D


def _np_softmax(x, axis):
    e = np.exp(x - x.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


@pytest.mark.parametrize("dim", [0, 1, 2, 7])
def test_oracle_softmax_matches_numpy_and_sums_to_one(oracle, dim):
    rng = np.random.default_rng(dim)
    shape = [3, 5, 4]
    x = rng.standard_normal(shape)
    axis = dim if dim < 3 else 2  # an out-of-range dim means the last one (softmax.rs:70)
    for dt in D.FLOATS:
        store = np.concatenate([D.encode([0.0], dt), D.encode(x.ravel(), dt)])  # offset 1, as the reference's fixtures
        got = D.decode(H.run_softmax(oracle, dt, shape, H.contiguous_strides(shape), 1, dim, store), dt).reshape(shape)
        want = _np_softmax(D.decode(D.encode(x.ravel(), dt), dt).reshape(shape), axis)
        tol = {"f64": 1e-12, "f32": 1e-6, "bf16": 3e-2, "f16": 4e-3}[dt.name]
        assert np.allclose(got, want, rtol=tol, atol=tol * 1e-2), dt.name
        assert np.allclose(got.sum(axis=axis), 1.0, atol=5e-2 if dt.name in ("bf16", "f16") else 1e-5)


def test_oracle_softmax_rows_of_the_reference_example(oracle):
    """The reference's own example input [[1,2,3],[4,5,6]] along dim 1: both rows give the same distribution."""
    x = np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    got = D.decode(H.run_softmax(oracle, D.F32, [2, 3], [3, 1], 0, 1, D.encode(x.ravel(), D.F32)), D.F32).reshape(2, 3)
    assert np.allclose(got[0], got[1], atol=1e-7) and np.all(np.diff(got[0]) > 0) and np.allclose(got.sum(axis=1), 1.0, atol=1e-6)
    # along dim 0: every column is softmax([a, a + 3])
    got0 = D.decode(H.run_softmax(oracle, D.F32, [2, 3], [3, 1], 0, 0, D.encode(x.ravel(), D.F32)), D.F32).reshape(2, 3)
    assert np.allclose(got0[0], 1.0 / (1.0 + np.exp(3.0)), rtol=1e-6) and np.all(got0[0] < got0[1])


NP_MODE = {"constant": "constant", "reflection": "reflect", "replication": "edge"}


@pytest.mark.parametrize("mode", ["constant", "reflection", "replication"])
def test_oracle_padding_agrees_with_numpy_pad(oracle, mode):
    """np.pad's constant / reflect / edge modes are the three paddings; the backward pass is the transpose of the
    forward gather, built here by padding an index array and scatter-adding."""
    rng = np.random.default_rng(len(mode))
    cases = [([11], [(3, 5)]), ([6, 9], [(2, 1), (4, 3)]), ([3, 5, 7], [(0, 2), (1, 0), (3, 3)])]
    for dt in (D.F64, D.F32, D.I32, D.U8):
        for shape, pads in cases:
            n = int(np.prod(shape))
            x = rng.integers(0, 50, n).astype(np.float64)
            store = D.encode(x, dt)
            kw = {"constant_values": 7} if mode == "constant" else {}
            want = np.pad(x.reshape(shape), pads, mode=NP_MODE[mode], **kw).ravel()
            got = H.run_pad(oracle, mode, dt, shape, H.contiguous_strides(shape), 0, pads, store, 7)
            assert np.array_equal(D.decode(got, dt).astype(np.float64), want), (mode, dt.name, shape)
            # a transposed view of the same data gives the padded transpose
            if len(shape) == 2:
                xt = np.ascontiguousarray(x.reshape(shape).T)       # stored transposed, viewed back as `shape`
                got_t = H.run_pad(oracle, mode, dt, shape, [1, shape[0]], 0, pads, D.encode(xt.ravel(), dt), 7)
                assert np.array_equal(D.decode(got_t, dt).astype(np.float64), want), (mode, dt.name, "transposed")
            # backward: where each output element was read from
            idx = np.arange(n, dtype=np.int64).reshape(shape)
            if mode == "constant":
                src = np.pad(idx, pads, mode="constant", constant_values=-1).ravel()
            else:
                src = np.pad(idx, pads, mode=NP_MODE[mode]).ravel()
            g = rng.integers(-20, 20, src.size).astype(np.float64) if dt is not D.U8 else rng.integers(0, 5, src.size).astype(np.float64)
            want_g = np.zeros(n)
            np.add.at(want_g, src[src >= 0], g[src >= 0])
            got_g = H.run_pad_backward(oracle, mode, dt, shape, H.contiguous_strides(shape), 0, pads, D.encode(g, dt), n)
            ref = want_g if dt is not D.U8 else np.mod(want_g, 256)
            assert np.array_equal(D.decode(got_g, dt).astype(np.float64), ref), (mode, dt.name, shape, "backward")


def test_oracle_fold_is_the_transpose_of_unfold(oracle):
    """fold(unfold view of x) multiplies every element by the number of windows that cover it, and fold of a dense
    gradient equals numpy's scatter-add over the window positions."""
    rng = np.random.default_rng(3)
    for shape, dim, size, step in (([23], 0, 5, 2), ([4, 17], 1, 4, 3), ([9, 6], 0, 3, 1)):
        st = H.contiguous_strides(shape)
        nwin = (shape[dim] - size) // step + 1
        dims = shape[:dim] + [nwin, size] + shape[dim + 1:]
        g = rng.integers(-9, 9, int(np.prod(dims))).astype(np.float64)
        fold_size = (nwin - 1) * step + size
        out_shape = shape[:dim] + [fold_size] + shape[dim + 1:]
        want = np.zeros(out_shape)
        gv = g.reshape(dims)
        for w in range(nwin):
            for p in range(size):
                sl = [slice(None)] * len(out_shape)
                sl[dim] = w * step + p
                src = [slice(None)] * len(dims)
                src[dim], src[dim + 1] = w, p
                want[tuple(sl)] += gv[tuple(src)]
        for dt in (D.F64, D.F32, D.I64):
            got = H.run_fold(oracle, dt, dims, H.contiguous_strides(dims), dim, dim + 1, fold_size, step, 0, D.encode(g, dt))
            assert np.array_equal(D.decode(got, dt).astype(np.float64), want.ravel()), (shape, dim, dt.name)


def _np_im2col(x, kh, kw, ph, pw, sh, sw):
    B, C, Hh, W = x.shape
    oh, ow = (Hh + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
    xp = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)))
    col = np.zeros((B, C, kh, kw, oh, ow))
    for i in range(kh):
        for j in range(kw):
            col[:, :, i, j] = xp[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw]
    return col, oh, ow


@pytest.mark.parametrize("geom", [(3, 3, 1, 1, 1, 1), (3, 3, 0, 0, 2, 2), (2, 5, 1, 2, 1, 3), (1, 1, 0, 0, 1, 1)], ids=str)
def test_oracle_im2col_col2im_agree_with_numpy(oracle, geom):
    """The reference pins conv only by shapes; this checks the restatement against an independent numpy
    formulation: col[b][c,kh,kw][oh,ow] = padded x at (oh*s - p + kh, ow*s - p + kw), and col2im as its transpose."""
    kh, kw, ph, pw, sh, sw = geom
    rng = np.random.default_rng(sum(geom))
    B, C, Hh, W = 2, 3, 9, 11
    x = rng.integers(-9, 9, (B, C, Hh, W)).astype(np.float64)
    col, oh, ow = _np_im2col(x, kh, kw, ph, pw, sh, sw)
    meta = H.conv_metadata(B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw)
    for dt in (D.F32, D.F64):
        got = H.run_im2col(oracle, dt, meta, col.size, D.encode(x.ravel(), dt))
        assert np.array_equal(D.decode(got, dt).astype(np.float64), col.ravel()), (geom, dt.name)
        # col2im of an arbitrary col = the transpose of the gather: scatter-add every col entry to its pixel
        g = rng.integers(-9, 9, col.shape).astype(np.float64)
        want = np.zeros((B, C, Hh + 2 * ph, W + 2 * pw))
        for i in range(kh):
            for j in range(kw):
                want[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw] += g[:, :, i, j]
        want = want[:, :, ph:ph + Hh, pw:pw + W]
        got = H.run_col2im(oracle, dt, meta, g.size, D.encode(g.ravel(), dt), x.size)
        assert np.array_equal(D.decode(got, dt).astype(np.float64), want.ravel()), (geom, dt.name, "col2im")
