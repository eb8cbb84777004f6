"""Shared test plumbing: one calling convention over two backends.

`OracleBackend` calls the CPU oracle (host pointers, host metadata); `CudaBackend` calls
libmaidenx_cuda.so exactly the way the reference's dispatch layer does (device buffers
from cuda_malloc, metadata uploaded with cuda_malloc + cuda_memcpy_h2d and freed after the
call).  The run_* helpers take the stored bits of whole underlying buffers plus the
metadata fields and return the output as a numpy array, so a parity test is
`run_x(oracle, ...)` vs `run_x(cuda, ...)` on the same arguments.
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from maidenx_b200 import dtypes as D  # noqa: E402
from maidenx_b200 import _signatures as sig  # noqa: E402

BOOL_OUT = set(sig.BINARY_BOOL + sig.UNARY_BOOL + sig.UNARY_CONST_BOOL)


def out_storage(op: str, dt: D.DType):
    return np.bool_ if op in BOOL_OUT else dt.np_storage


class OracleBackend:
    name = "oracle"

    def __init__(self):
        from oracle import binding
        self.b = binding
        binding.load()

    def call(self, op, dt, metadata, build_args):
        """build_args(put, META) -> (arg list, outputs dict name -> (handle, np dtype, count))."""
        keep = []

        def put(arr):
            a = np.ascontiguousarray(arr).copy()
            keep.append(a)
            return a.ctypes.data, a

        m = None if metadata is None else np.asarray(metadata, dtype=np.uint64)
        mptr = None if m is None else m.ctypes.data
        args, outs = build_args(put, mptr)
        self.b.op(op, dt.name)(*args)
        return {k: h.copy() for k, (h, _, _) in outs.items()}


class CudaBackend:
    name = "cuda"

    def __init__(self, metadata_on_host: bool = False):
        from maidenx_b200 import device
        self.dev = device
        self.metadata_on_host = metadata_on_host

    def call(self, op, dt, metadata, build_args):
        bufs = []

        def put(arr):
            b = self.dev.CudaBuffer.from_host(np.ascontiguousarray(arr))
            bufs.append(b)
            return b.ptr, b

        args, outs = build_args(put, "META")
        try:
            self.dev.dispatch(op, dt.name, metadata, *args, metadata_on_host=self.metadata_on_host)
            self.dev.synchronize()
            res = {k: h.to_host(npdt, cnt) for k, (h, npdt, cnt) in outs.items()}
        finally:
            for b in bufs:
                b.free()
        return res


def _sz(x):
    return ctypes.c_size_t(int(x))


def contiguous_strides(dims):
    st, acc = [], 1
    for d in reversed(dims):
        st.append(acc)
        acc *= d
    return list(reversed(st))


def numel(dims):
    n = 1
    for d in dims:
        n *= d
    return n


# ---------------------------------------------------------------------------------------
def run_binary(be, op, dt, dims, lstr, rstr, loff, roff, lhs_store, rhs_store, null_meta=False, out_fill=None):
    n = numel(dims)
    nd = len(dims)
    meta = None if null_meta else list(dims) + list(lstr) + list(rstr) + [loff, roff]
    ost = out_storage(op, dt)
    out0 = np.zeros(n, dtype=ost) if out_fill is None else np.full(n, out_fill, dtype=ost)

    def build(put, META):
        lp, _ = put(lhs_store)
        rp, _ = put(rhs_store)
        op_, oh = put(out0)
        return [_sz(n), _sz(nd), META, lp, rp, op_], {"out": (oh, ost, n)}

    return be.call(op, dt, meta, build)["out"]


def run_binary_inplace(be, op, dt, dims, lstr, rstr, loff, roff, lhs_store, rhs_store, null_meta=False):
    n = numel(dims)
    nd = len(dims)
    meta = None if null_meta else list(dims) + list(lstr) + list(rstr) + [loff, roff]

    def build(put, META):
        lp, lh = put(lhs_store)
        rp, _ = put(rhs_store)
        return [_sz(n), _sz(nd), META, lp, rp], {"lhs": (lh, dt.np_storage, len(lhs_store))}

    return be.call(op, dt, meta, build)["lhs"]


def run_unary(be, op, dt, dims, strides, off, in_store, scalar=None, null_meta=False):
    n = numel(dims)
    nd = len(dims)
    meta = None if null_meta else list(dims) + list(strides) + [off]
    ost = out_storage(op, dt)

    def build(put, META):
        ip, _ = put(in_store)
        op_, oh = put(np.zeros(n, dtype=ost))
        args = [_sz(n), _sz(nd), META, ip]
        if scalar is not None:
            args.append(D.scalar_arg(scalar, dt))
        args.append(op_)
        return args, {"out": (oh, ost, n)}

    return be.call(op, dt, meta, build)["out"]


def run_reduce(be, op, dt, dims, strides, red_lens, red_strides, off, in_store, out_fill=None):
    n = numel(dims)
    out_n = n
    for l in red_lens:
        out_n //= l
    meta = list(dims) + list(strides) + list(red_lens) + list(red_strides) + [off]
    # the caller's buffer is deliberately dirty: ops must overwrite, not accumulate
    out0 = np.full(max(out_n, 1), 7 if out_fill is None else out_fill).astype(dt.np_storage)

    def build(put, META):
        ip, _ = put(in_store)
        op_, oh = put(out0)
        return [_sz(n), _sz(len(dims)), _sz(len(red_lens)), META, ip, op_], {"out": (oh, dt.np_storage, out_n)}

    return be.call(op, dt, meta, build)["out"]


def run_sum_to_shape(be, dt, dims, strides, out_dims, off, in_store):
    n = numel(dims)
    out_n = numel(out_dims)
    meta = list(dims) + list(strides) + list(out_dims) + [off]
    out0 = np.full(max(out_n, 1), 7).astype(dt.np_storage)

    def build(put, META):
        ip, _ = put(in_store)
        op_, oh = put(out0)
        return [_sz(n), _sz(len(dims)), META, ip, op_], {"out": (oh, dt.np_storage, out_n)}

    return be.call("sum_to_shape", dt, meta, build)["out"]


def pad_metadata(in_dims, in_strides, off, pads):
    """crates/maidenx_tensor/src/ops/padding.rs:272-294."""
    out_dims = [d + a + b for d, (a, b) in zip(in_dims, pads)]
    flat = [v for ab in pads for v in ab]
    return list(in_dims) + list(in_strides) + [off] + out_dims + flat, out_dims


def run_pad(be, mode, dt, in_dims, in_strides, off, pads, in_store, value=None):
    """mode: constant | reflection | replication.  Returns the padded tensor (dense)."""
    meta, out_dims = pad_metadata(in_dims, in_strides, off, pads)
    n_in, n_out = numel(in_dims), numel(out_dims)
    out0 = np.full(max(n_out, 1), 7).astype(dt.np_storage)  # dirty: the op must overwrite

    def build(put, META):
        ip, _ = put(in_store)
        op_, oh = put(out0)
        args = [_sz(n_in), _sz(n_out), _sz(len(in_dims)), META, ip, op_]
        if mode == "constant":
            args.append(D.scalar_arg(value, dt))
        return args, {"out": (oh, dt.np_storage, n_out)}

    return be.call(f"pad_with_{mode}", dt, meta, build)["out"]


def run_pad_backward(be, mode, dt, in_dims, in_strides, off, pads, grad_out_store, grad_in_len):
    """Returns the whole grad_in buffer (grad_in_len elements; the op writes [off, off + numel(in_dims)))."""
    meta, out_dims = pad_metadata(in_dims, in_strides, off, pads)
    n_in, n_out = numel(in_dims), numel(out_dims)
    gi0 = np.full(max(grad_in_len, 1), 7).astype(dt.np_storage)

    def build(put, META):
        gp, _ = put(grad_out_store)
        ip, ih = put(gi0)
        return [_sz(n_in), _sz(n_out), _sz(len(in_dims)), META, gp, ip], {"grad_in": (ih, dt.np_storage, grad_in_len)}

    return be.call(f"pad_with_{mode}_backward", dt, meta, build)["grad_in"]


def run_fold(be, dt, dims, strides, fold_dim, window_dim, fold_size, step, off, in_store):
    """crates/maidenx_tensor/src/ops/reduction.rs:745-769: [dims | strides | fold_dim, window_dim, fold_size, step, window_size, offset]."""
    n = numel(dims)
    meta = list(dims) + list(strides) + [fold_dim, window_dim, fold_size, step, dims[window_dim], off]
    out_n = 1
    for d, ext in enumerate(dims):
        if d == window_dim:
            continue
        out_n *= fold_size if d == fold_dim else ext
    out0 = np.full(max(out_n, 1), 7).astype(dt.np_storage)

    def build(put, META):
        ip, _ = put(in_store)
        op_, oh = put(out0)
        return [_sz(n), _sz(len(dims)), META, ip, op_], {"out": (oh, dt.np_storage, out_n)}

    return be.call("fold", dt, meta, build)["out"]


def run_softmax(be, dt, dims, strides, off, dim, in_store):
    n = numel(dims)
    meta = list(dims) + list(strides) + [off]
    out0 = np.full(max(n, 1), 7).astype(dt.np_storage)

    def build(put, META):
        ip, _ = put(in_store)
        op_, oh = put(out0)
        return [_sz(n), _sz(len(dims)), _sz(dim), META, ip, op_], {"out": (oh, dt.np_storage, n)}

    return be.call("softmax", dt, meta, build)["out"]


def matmul_metadata(out_shape, a_shape, b_shape, a_strides, b_strides, a_off, b_off):
    """crates/maidenx_tensor/src/ops/matmul.rs:227-264."""
    return [len(out_shape), len(a_shape), len(b_shape)] + list(out_shape) + list(a_shape) + list(b_shape) + \
        list(a_strides) + list(b_strides) + [a_off, b_off]


def run_matmul(be, dt, meta, num_els, a_store, b_store):
    def build(put, META):
        ap, _ = put(a_store)
        bp, _ = put(b_store)
        cp, ch = put(np.full(max(num_els, 1), 7).astype(dt.np_storage))
        return [_sz(num_els), META, ap, bp, cp], {"c": (ch, dt.np_storage, num_els)}

    return be.call("matmul", dt, meta, build)["c"]


def run_matmul_backward(be, dt, meta, num_els_a, num_els_b, g_store, a_store, b_store, want_a=True, want_b=True):
    def build(put, META):
        gp, _ = put(g_store)
        ap, _ = put(a_store)
        bp, _ = put(b_store)
        outs = {}
        gap = gbp = None
        if want_a:
            gap, gah = put(np.full(max(num_els_a, 1), 7).astype(dt.np_storage))
            outs["ga"] = (gah, dt.np_storage, num_els_a)
        if want_b:
            gbp, gbh = put(np.full(max(num_els_b, 1), 7).astype(dt.np_storage))
            outs["gb"] = (gbh, dt.np_storage, num_els_b)
        return [_sz(num_els_a), _sz(num_els_b), META, gp, ap, bp, gap, gbp], outs

    return be.call("matmul_backward", dt, meta, build)


def conv_metadata(B, C, H, W, kh, kw, oh, ow, ph, pw, sh, sw):
    return [B, C, H, W, kh, kw, oh, ow, ph, pw, sh, sw]


def run_im2col(be, dt, meta, num_els, x_store, col_len=None):
    col_len = num_els if col_len is None else col_len

    def build(put, META):
        xp, _ = put(x_store)
        cp, ch = put(np.full(max(col_len, 1), 7).astype(dt.np_storage))
        return [_sz(num_els), META, xp, cp], {"col": (ch, dt.np_storage, col_len)}

    return be.call("conv2d_im2col", dt, meta, build)["col"]


def run_col2im(be, dt, meta, num_els, col_store, out_len):
    def build(put, META):
        cp, _ = put(col_store)
        op_, oh = put(np.full(max(out_len, 1), 7).astype(dt.np_storage))
        return [_sz(num_els), META, cp, op_], {"out": (oh, dt.np_storage, out_len)}

    return be.call("conv2d_col2im", dt, meta, build)["out"]


# ---------------------------------------------------------------------------------------
# seeded inputs
# ---------------------------------------------------------------------------------------
def random_store(rng, dt: D.DType, count: int, dist: str = "uniform", lo=-1.0, hi=1.0):
    """Stored bits of `count` seeded values: U(lo,hi) or N(0,1) for floats, U[lo,hi] ints otherwise."""
    if dt.kind == "float":
        v = rng.uniform(lo, hi, count) if dist == "uniform" else rng.standard_normal(count)
        return D.encode(v.astype(np.float32) if dt is not D.F64 else v, dt)
    if dt.kind == "bool":
        return rng.integers(0, 2, count).astype(np.bool_)
    info = np.iinfo(dt.np_storage)
    a, b = max(int(lo), info.min), min(int(hi), info.max)
    return rng.integers(a, b + 1, count).astype(dt.np_storage)


def full_range_store(rng, dt: D.DType, count: int):
    """Integers over the type's whole range (exercises saturation); floats N(0,1)*10 with specials."""
    if dt.kind in ("uint", "sint"):
        info = np.iinfo(dt.np_storage)
        v = rng.integers(info.min, info.max, count, dtype=dt.np_storage, endpoint=True)
        edge = np.array([info.min, info.max, 0, 1, info.max - 1] + ([-1, info.min + 1] if dt.kind == "sint" else []), dtype=dt.np_storage)
        k = min(count, len(edge) * 3)
        v[:k] = np.resize(edge, k)
        return rng.permutation(v)
    if dt.kind == "bool":
        return rng.integers(0, 2, count).astype(np.bool_)
    v = rng.standard_normal(count) * 10.0
    specials = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 65504.0, 1e-8, 3.0e38])
    k = min(count, len(specials) * 2)
    v[:k] = np.resize(specials, k)
    v = rng.permutation(v)
    return D.encode(v.astype(np.float32) if dt is not D.F64 else v, dt)


def assert_same(op, dt, got, ref, float_rel=0.0, what="", scale=None):
    """Bit-exact for bool / integer outputs; for float outputs exact when float_rel == 0
    (NaNs compare equal as a class), else |got - ref| <= float_rel * max(|ref|, scale).
    `scale` (scalar or per-element) is the magnitude of the intermediate a formula cancels
    against: 0.5*x*(1 + tanh(t)) loses |x| * eps when tanh(t) is near -1, alpha*(exp(x) - 1)
    loses alpha * eps near x = 0; the relative bound is taken against that magnitude."""
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    if got.dtype == np.bool_ or dt.kind in ("uint", "sint", "bool"):
        bad = np.nonzero(got != ref)[0]
        assert bad.size == 0, f"{what} {op}_{dt.name}: {bad.size} mismatches, first at {bad[:5]}: got {got[bad[:5]]} want {ref[bad[:5]]}"
        return
    g, r = D.decode(got, dt), D.decode(ref, dt)
    nan_g, nan_r = np.isnan(g), np.isnan(r)
    assert np.array_equal(nan_g, nan_r), f"{what} {op}_{dt.name}: NaN pattern differs"
    ok = ~nan_g
    sc = np.full(g.shape, 1e-30) if scale is None else np.broadcast_to(np.abs(np.asarray(scale, dtype=np.float64)), g.shape)
    g, r, sc = g[ok], r[ok], sc[ok]
    inf = np.isinf(r)
    assert np.array_equal(g[inf], r[inf]), f"{what} {op}_{dt.name}: infinities differ"
    assert not np.isinf(g[~inf]).any(), f"{what} {op}_{dt.name}: unexpected infinity"
    g, r, sc = g[~inf], r[~inf], sc[~inf]
    if float_rel == 0.0:
        bad = np.nonzero(g != r)[0]
    else:
        bad = np.nonzero(np.abs(g - r) > float_rel * np.maximum(np.abs(r), np.maximum(sc, 1e-30)))[0]
    assert bad.size == 0, f"{what} {op}_{dt.name}: {bad.size} mismatches (rel {float_rel}), first: got {g[bad[:5]]} want {r[bad[:5]]}"
