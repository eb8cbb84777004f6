"""Conv2d forward / backward composed op by op through the test harness, on either backend.

`compose(be, ...)` issues the same op calls as maidenx_b200/csrc/conv2d_layer.cu (mode 0: the calls of
crates/maidenx_nn/src/layers/conv.rs:185-307,333-420 taken literally; mode 1: the same ops used consistently), so
running it on the CPU oracle gives the reference-side answer for the layer.  The reference's `contiguous()` of a
strided view is a host-side element walk (crates/maidenx_tensor/src/f.rs:11-40); numpy's strided gather stands in
for it here.  `direct_conv_f64` is an independent float64 convolution (no im2col, no matmul) for mode 1.
"""
import numpy as np
from numpy.lib.stride_tricks import as_strided

import harness as H
from maidenx_b200 import dtypes as D


def geometry(B, C, Hh, W, Co, kh, kw, sh, sw, ph, pw):
    oh = (Hh + 2 * ph - kh) // sh + 1
    ow = (W + 2 * pw - kw) // sw + 1
    return oh, ow, oh * ow, C * kh * kw


def _gather(store, dims, strides, off=0):
    """contiguous() of a strided view over `store`."""
    es = store.dtype.itemsize
    v = as_strided(store[off:], shape=dims, strides=[s * es for s in strides])
    return np.ascontiguousarray(v).reshape(-1)


def _sum_dim(be, dt, dims, dim, store):
    st = H.contiguous_strides(dims)
    return H.run_reduce(be, "sum", dt, dims, st, [dims[dim]], [st[dim]], 0, store)


def compose(be, dt, mode, shape, x, w, bias, grad_out):
    """Returns dict(out, grad_x, grad_w, grad_bias, cols).  All arrays are stored bits (dt.np_storage), flat."""
    B, C, Hh, W, Co, kh, kw, sh, sw, ph, pw = shape
    oh, ow, P, K = geometry(*shape)
    ncol = B * P * K
    res = {}
    if mode == 0:
        cm = H.conv_metadata(B, C, Hh, W, kh, kw, oh, ow, sh, sw, ph, pw)  # stride where the kernels read padding
        cols = H.run_im2col(be, dt, cm, ncol, x)
        M = B * P
        flat = H.run_matmul(be, dt, H.matmul_metadata([M, Co], [M, K], [K, Co], [K, 1], [1, K], 0, 0), M * Co, cols, w)
        vs = [P * Co, 1, ow * Co, Co]
        if bias is not None:
            res["out"] = H.run_binary(be, "add", dt, [B, Co, oh, ow], vs, [0, 1, 0, 0], 0, 0, flat, bias)
        else:
            res["out"] = _gather(flat, [B, Co, oh, ow], vs)
        gflat = _gather(grad_out, [B, oh, ow, Co], [Co * P, ow, 1, P])
        gcols = H.run_matmul(be, dt, H.matmul_metadata([M, K], [M, Co], [Co, K], [Co, 1], [K, 1], 0, 0), M * K, gflat, w)
        res["grad_x"] = H.run_col2im(be, dt, cm, B * C * Hh * W, gcols, B * C * Hh * W)
        res["grad_w"] = H.run_matmul(be, dt, H.matmul_metadata([K, Co], [K, M], [M, Co], [1, K], [Co, 1], 0, 0), K * Co, cols, gflat)
    else:
        cm = H.conv_metadata(B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw)
        cols = H.run_im2col(be, dt, cm, ncol, x)
        out = H.run_matmul(be, dt, H.matmul_metadata([B, Co, P], [B, Co, K], [B, K, P], [0, K, 1], [K * P, P, 1], 0, 0), B * Co * P, w, cols)
        if bias is not None:
            out = H.run_binary_inplace(be, "add_inplace", dt, [B, Co, P], [Co * P, P, 1], [0, 1, 0], 0, 0, out, bias)
        res["out"] = out
        gcols = H.run_matmul(be, dt, H.matmul_metadata([B, K, P], [B, K, Co], [B, Co, P], [0, 1, K], [Co * P, P, 1], 0, 0), B * K * P, w, grad_out)
        res["grad_x"] = H.run_col2im(be, dt, cm, B * K * P, gcols, B * C * Hh * W)
        gw = H.run_matmul(be, dt, H.matmul_metadata([B, Co, K], [B, Co, P], [B, P, K], [Co * P, P, 1], [K * P, 1, P], 0, 0), B * Co * K, grad_out, cols)
        res["grad_w"] = _sum_dim(be, dt, [B, Co, K], 0, gw)
    t = _sum_dim(be, dt, [B, Co, oh, ow], 3, grad_out)
    t = _sum_dim(be, dt, [B, Co, oh], 2, t)
    res["grad_bias"] = _sum_dim(be, dt, [B, Co], 0, t)
    res["cols"] = cols
    return res


def direct_conv_f64(shape, x, w, bias, grad_out):
    """Float64 convolution and its gradients straight from the definition (loops over the kernel window only)."""
    B, C, Hh, W, Co, kh, kw, sh, sw, ph, pw = shape
    oh, ow, _, _ = geometry(*shape)
    x = np.asarray(x, np.float64).reshape(B, C, Hh, W)
    w = np.asarray(w, np.float64).reshape(Co, C, kh, kw)
    g = np.asarray(grad_out, np.float64).reshape(B, Co, oh, ow)
    xp = np.zeros((B, C, Hh + 2 * ph, W + 2 * pw))
    xp[:, :, ph:ph + Hh, pw:pw + W] = x
    out = np.zeros((B, Co, oh, ow))
    gxp = np.zeros_like(xp)
    gw = np.zeros_like(w)
    for i in range(kh):
        for j in range(kw):
            win = xp[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw]            # [B, C, oh, ow]
            out += np.einsum("bchw,oc->bohw", win, w[:, :, i, j])
            gw[:, :, i, j] = np.einsum("bohw,bchw->oc", g, win)
            gxp[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw] += np.einsum("bohw,oc->bchw", g, w[:, :, i, j])
    if bias is not None:
        out += np.asarray(bias, np.float64).reshape(1, Co, 1, 1)
    return {"out": out.reshape(-1), "grad_x": gxp[:, :, ph:ph + Hh, pw:pw + W].reshape(-1), "grad_w": gw.reshape(-1),
            "grad_bias": g.sum(axis=(0, 2, 3))}


def run_layer(dt, mode, shape, x, w, bias, grad_out):
    """The library's own composition (mx_conv2d_forward / backward) through the C ABI, device buffers."""
    import ctypes
    from maidenx_b200 import _lib, device
    lib = _lib.load()
    conv = _lib.MxConv2d(*shape)
    ncol, nout = lib.mx_conv2d_cols_elems(ctypes.byref(conv)), lib.mx_conv2d_output_elems(ctypes.byref(conv))
    B, C, Hh, W, Co, kh, kw = shape[:7]
    K = C * kh * kw
    st = dt.np_storage
    dirty = lambda n: np.full(max(n, 1), 7).astype(st)  # noqa: E731  outputs and scratch start dirty on purpose
    fwd_ws = lib.mx_conv2d_workspace_elems(ctypes.byref(conv), mode, 0)
    bwd_ws = lib.mx_conv2d_workspace_elems(ctypes.byref(conv), mode, 1)
    bufs = {k: device.CudaBuffer.from_host(v) for k, v in dict(
        x=x, w=w, g=grad_out, cols=dirty(ncol), ws=dirty(max(fwd_ws, bwd_ws)), out=dirty(nout), gx=dirty(x.size), gw=dirty(K * Co), gb=dirty(Co)).items()}
    if bias is not None:
        bufs["b"] = device.CudaBuffer.from_host(bias)
    try:
        fwd, bwd = _lib.conv2d(dt.name)
        fwd(ctypes.byref(conv), mode, bufs["x"].ptr, bufs["w"].ptr, bufs["b"].ptr if bias is not None else None, bufs["cols"].ptr, bufs["ws"].ptr,
            bufs["out"].ptr)
        bwd(ctypes.byref(conv), mode, bufs["g"].ptr, bufs["w"].ptr, bufs["cols"].ptr, bufs["ws"].ptr, bufs["gx"].ptr, bufs["gw"].ptr, bufs["gb"].ptr)
        device.synchronize()
        err = device.last_error()
        assert err is None, err
        return {"out": bufs["out"].to_host(st, nout), "grad_x": bufs["gx"].to_host(st, x.size), "grad_w": bufs["gw"].to_host(st, K * Co),
                "grad_bias": bufs["gb"].to_host(st, Co), "cols": bufs["cols"].to_host(st, ncol)}
    finally:
        for b in bufs.values():
            b.free()
