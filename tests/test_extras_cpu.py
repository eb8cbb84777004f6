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
