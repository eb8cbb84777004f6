"""Replays the known-answer vectors of the reference's own tests
(tests/golden/reference_vectors.json, lifted from crates/maidenx_tensor/tests/*.rs and
crates/maidenx_nn/src/losses/mse.rs) on both backends: on the CPU oracle (runs without a GPU
and pins the oracle) and, marked gpu, on the CUDA library through its C ABI.

The reference's tests work at the Tensor level; a vector is replayed at the op level only
where the Tensor method hands the same dtype straight to the backend op.  The Tensor-level
promotions that break that one-to-one mapping are listed in PROMOTED below with the
reference lines that perform them.
"""
import json
from pathlib import Path

import numpy as np
import pytest

import harness as H
from maidenx_b200 import dtypes as D

GOLD = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())
INT_NAMES = {d.name for d in D.INTS}


@pytest.fixture(params=["oracle", pytest.param("cuda", marks=pytest.mark.gpu)])
def be(request):
    """The backend a vector is replayed on."""
    return request.getfixturevalue(request.param)

# Tensor methods that change dtype before calling the backend for integer inputs
# (crates/maidenx_tensor/src/ops/unary.rs): sqrt and every transcendental promote integers to
# F32 (:149-155 and the same pattern through :733-740); div / div_scalar / leaky_relu / elu do
# too (crates/maidenx_tensor/src/ops/binary.rs:172-178, unary.rs:909-915,1084-1090,1129-1135);
# neg converts unsigned to signed (:8-15) and abs clones unsigned inputs (:45-55).
PROMOTED_INT = {"sqrt", "relu", "sigmoid", "tanh", "gelu", "sin", "cos", "tan", "ln", "log10", "log2", "exp", "exp10",
                "exp2", "softplus", "recip", "div", "div_inplace", "div_scalar", "leaky_relu", "elu"}
UNSIGNED_SKIP = {"neg", "abs"}
TRANSCENDENTAL = {"sigmoid", "tanh", "gelu", "sin", "cos", "tan", "ln", "log10", "log2", "exp", "exp10", "exp2", "softplus",
                  "pow", "elu", "sqrt", "recip"}
# Non-integer scalars promote the tensor to F32 (unary.rs:794-801 and siblings)
METHOD_TO_OP = {"add_": "add_inplace", "sub_": "sub_inplace", "mul_": "mul_inplace", "div_": "div_inplace"}


def _cases(kind):
    for rec in GOLD[kind]:
        op = METHOD_TO_OP.get(rec["method"], rec["method"])
        for name in rec["dtypes"]:
            dt = D.BY_NAME[name]
            if name in INT_NAMES:
                if op in PROMOTED_INT:
                    continue
                if op in UNSIGNED_SKIP and dt.kind == "uint":
                    continue
                if "scalar" in rec and isinstance(rec["scalar"], float) and not float(rec["scalar"]).is_integer():
                    continue
            yield pytest.param(rec, op, dt, id=f"{op}-{name}-{rec['cite'].split(':')[-1]}")


def _val(x):
    return {"inf": np.inf, "-inf": -np.inf, "nan": np.nan}.get(x, x) if isinstance(x, str) else x


def _padded(values, dt):
    """The reference's fixtures: one default element either side, viewed from element 1
    (crates/maidenx_tensor/tests/utils/mod.rs:30-37)."""
    v = [_val(x) for x in values]
    return D.encode(np.array([0] + v + [0], dtype=np.float64 if dt.kind == "float" else None), dt)


def _check(rec, got, dt, op, be=None):
    exp = np.array([_val(x) for x in rec["expected"]], dtype=np.float64)
    g = D.decode(got, dt).astype(np.float64)
    tol = rec["tol"]
    if "exact" in tol:
        if dt.name in ("bf16", "f16"):
            assert np.allclose(g, exp, atol=0.1), (op, dt.name, g, exp)
        elif be is not None and be.name == "cuda" and dt.kind == "float" and op in TRANSCENDENTAL:
            # the device's math functions are held to the stated f32 tolerance, not to libm's bits
            assert np.allclose(g, exp, rtol=1e-5 if dt.name == "f32" else 1e-12, atol=1e-6 if dt.name == "f32" else 1e-12, equal_nan=True), (op, dt.name, g, exp)
        else:
            # f32 values printed in the test source compare equal after rounding to f32
            assert np.array_equal(g.astype(np.float32), exp.astype(np.float32)), (op, dt.name, g, exp)
    elif "abs" in tol:
        assert np.all(np.abs(g - exp) < tol["abs"]), (op, dt.name, g, exp)
    else:
        assert np.all(np.abs(g - exp) < tol["rel"] * np.abs(exp)), (op, dt.name, g, exp)


@pytest.mark.parametrize("rec,op,dt", list(_cases("binary")))
def test_binary_golden(be, rec, op, dt):
    n = len(rec["lhs"])
    lhs, rhs = _padded(rec["lhs"], dt), _padded(rec["rhs"], dt)
    if rec["inplace"]:
        got = H.run_binary_inplace(be, op, dt, [n], [1], [1], 1, 1, lhs, rhs)[1:-1]
    else:
        got = H.run_binary(be, op, dt, [n], [1], [1], 1, 1, lhs, rhs)
    _check(rec, got, dt, op, be)


@pytest.mark.parametrize("rec,op,dt", list(_cases("unary")))
def test_unary_golden(be, rec, op, dt):
    n = len(rec["lhs"])
    got = H.run_unary(be, op, dt, [n], [1], 1, _padded(rec["lhs"], dt), scalar=rec.get("scalar"))
    _check(rec, got, dt, op, be)


def _red_dtypes(classes):
    if classes == "int":
        return D.INTS
    if classes == "float":
        return D.FLOATS
    return D.ARITH


@pytest.mark.parametrize("rec", GOLD["reduction"], ids=lambda r: f"{r['op']}-{r['shape']}-{r['arg']}")
def test_reduction_golden(be, rec):
    for dt in _red_dtypes(rec["classes"]):
        if rec["op"] == "mean" and dt.kind != "float":
            continue
        store = _padded(rec["input"], dt)
        shape = rec["shape"]
        strides = H.contiguous_strides(shape)
        if rec["op"] == "sum_to_shape":
            got = H.run_sum_to_shape(be, dt, shape, strides, rec["arg"], 1, store)
        else:
            dim = rec["arg"]  # metadata as built by crates/maidenx_tensor/src/ops/reduction.rs:722-733
            got = H.run_reduce(be, rec["op"], dt, shape, strides, [shape[dim]], [strides[dim]], 1, store)
        g = D.decode(got, dt).astype(np.float64)
        assert np.allclose(g, np.array(rec["expected"], dtype=np.float64), atol=0.1 if dt.name in ("bf16", "f16") else 0), (dt.name, g)


def _unified(a_shape, b_shape):
    """Shapes/strides as Tensor::matmul prepares them (crates/maidenx_tensor/src/ops/matmul.rs:161-264)
    for the rank combinations the reference tests use (no leading-dim broadcast)."""
    a_sh = [1] + a_shape if len(a_shape) == 1 else list(a_shape)
    b_sh = b_shape + [1] if len(b_shape) == 1 else list(b_shape)
    out = a_sh[:-1] + [b_sh[-1]]
    return a_sh, b_sh, out


@pytest.mark.parametrize("rec", GOLD["matmul"], ids=lambda r: f"{r['a_shape']}x{r['b_shape']}")
def test_matmul_golden(be, rec):
    for dt in D.ARITH:
        a_sh, b_sh, out = _unified(rec["a_shape"], rec["b_shape"])
        meta = H.matmul_metadata(out, a_sh, b_sh, H.contiguous_strides(a_sh), H.contiguous_strides(b_sh), 1, 1)
        a, b = _padded(rec["a"], dt), _padded(rec["b"], dt)
        tol = 0.5 if dt.name in ("bf16", "f16") else 0
        if dt.name == "u8" or dt.name == "i8":
            pass  # Tensor::matmul widens 8-bit inputs (matmul.rs:18-27); at the op level they wrap
        c = H.run_matmul(be, dt, meta, H.numel(out), a, b)
        exp = np.array(rec["c"], dtype=np.float64)
        if dt.size == 1:
            exp = exp.astype(np.int64).astype(dt.np_storage).astype(np.float64)  # wrapping arithmetic
        assert np.allclose(D.decode(c, dt).astype(np.float64), exp, atol=tol), (dt.name, c)
        # backward of sum(C): grad_output = ones (crates/maidenx_tensor/src/lib.rs:293-323)
        g = D.encode(np.ones(H.numel(out)), dt)
        res = H.run_matmul_backward(be, dt, meta, len(rec["a"]), len(rec["b"]), g, a, b)
        for key, want in (("ga", rec["grad_a"]), ("gb", rec["grad_b"])):
            w = np.array(want, dtype=np.float64)
            assert np.allclose(D.decode(res[key], dt).astype(np.float64), w, atol=tol), (dt.name, key, res[key])


def test_mse_golden(be):
    """MSE forward/backward composed from ops the way crates/maidenx_nn/src/losses/mse.rs:21-29 and the
    autograd closures (crates/maidenx_tensor/src/ops/unary.rs:1066-1076, reduction.rs:52-71) do."""
    rec = GOLD["mse"]
    dt = D.F32
    pred, target = D.encode(rec["pred"], dt), D.encode(rec["target"], dt)
    n = len(rec["pred"])
    diff = H.run_binary(be, "sub", dt, [n], [1], [1], 0, 0, pred, target)
    sq = H.run_unary(be, "pow", dt, [n], [1], 0, diff, scalar=2.0)
    s = H.run_reduce(be, "sum", dt, [n], [1], [n], [1], 0, sq)
    loss = H.run_unary(be, "div_scalar", dt, [], [], 0, s, scalar=float(n))
    assert loss[0] == np.float32(rec["loss"])
    # d loss / d pred = (1/n) * 2 * diff^(2-1)
    g = H.run_unary(be, "div_scalar", dt, [], [], 0, np.ones(1, np.float32), scalar=float(n))
    gb = np.full(n, g[0], np.float32)  # broadcast of the scalar gradient
    p1 = H.run_unary(be, "pow", dt, [n], [1], 0, diff, scalar=1.0)
    p2 = H.run_unary(be, "mul_scalar", dt, [n], [1], 0, p1, scalar=2.0)
    grad = H.run_binary(be, "mul", dt, [n], [1], [1], 0, 0, gb, p2)
    assert np.allclose(grad, np.array(rec["grad"], np.float32), rtol=1e-6)


@pytest.mark.parametrize("rec", GOLD["padding"], ids=lambda r: f"{r['mode']}-{r['shape']}-{r['pads']}")
def test_padding_golden(be, rec):
    """Values from crates/maidenx_tensor/tests/ops_padding.rs; the gradient is the backward of sum(padded),
    i.e. the padding's backward applied to ones."""
    for dt in D.ARITH:
        if rec["value"] is not None and rec["value"] != int(rec["value"]) and dt.kind != "float":
            continue  # 9.9 truncates to 9 for integer dtypes in the reference's test; the float arm is the golden one
        shape, pads = rec["shape"], [tuple(p) for p in rec["pads"]]
        store = _padded(rec["input"], dt)
        got = H.run_pad(be, rec["mode"], dt, shape, H.contiguous_strides(shape), 1, pads, store, rec["value"])
        tol = 0.1 if dt.name in ("bf16", "f16") else (1e-6 if dt.name == "f32" else 0)
        assert np.allclose(D.decode(got, dt).astype(np.float64), np.array(rec["expected"]), atol=tol), (dt.name, got)
        if rec["grad"] is not None:
            n_out = len(rec["expected"])
            gi = H.run_pad_backward(be, rec["mode"], dt, shape, H.contiguous_strides(shape), 0, pads, D.encode(np.ones(n_out), dt), len(rec["input"]))
            assert np.allclose(D.decode(gi, dt).astype(np.float64), np.array(rec["grad"]), atol=tol), (dt.name, gi)


@pytest.mark.parametrize("rec", GOLD["fold"], ids=lambda r: f"{r['shape']}-dim{r['dim']}")
def test_fold_golden(be, rec):
    """crates/maidenx_tensor/tests/ops_reduction.rs:484-531: x.unfold(dim, size, step).fold(dim, size, step)."""
    for dt in D.ARITH:
        shape, dim, size, step = rec["shape"], rec["dim"], rec["size"], rec["step"]
        st = H.contiguous_strides(shape)
        nwin = (shape[dim] - size) // step + 1
        dims = shape[:dim] + [nwin, size] + shape[dim + 1:]      # the unfolded view (crates/maidenx_core/src/layout.rs:193-250):
        strides = st[:dim] + [step * st[dim], st[dim]] + st[dim + 1:]  # window count, then the window right behind it
        got = H.run_fold(be, dt, dims, strides, dim, dim + 1, shape[dim], step, 1, _padded(rec["input"], dt))
        tol = 0.1 if dt.name in ("bf16", "f16") else 0
        assert np.allclose(D.decode(got, dt).astype(np.float64), np.array(rec["expected"]), atol=tol), (dt.name, got)
