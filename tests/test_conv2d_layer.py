"""Conv2d as a whole: im2col + matmul forward, matmul + col2im / matmul / sums backward.

CPU (no GPU needed): the oracle, composed op by op in the consistent ("direct") way, is a convolution — checked
against an independent float64 convolution, which is a second, formulation-independent pin of the oracle's
im2col / col2im (the reference's own tests only check Conv2d shapes, crates/maidenx_nn/src/layers/conv.rs:422-471).
GPU: the library's composition (mx_conv2d_forward / backward through the C ABI) against the oracle composed with
the same calls, for the literal reference call sequence (mode 0) and the direct one (mode 1), and mode 1 against
the float64 convolution.  Tolerances: f32 1e-4 and bf16 / f16 2e-2 of max(|ref|, sqrt(terms)).
"""
import numpy as np
import pytest

import conv2d_compose as CC
import harness as H
from maidenx_b200 import dtypes as D

# B, C, H, W, Cout, kh, kw, sh, sw, ph, pw
SMALL = [
    (2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1),
    (3, 2, 7, 9, 5, 3, 2, 2, 1, 1, 0),
    (1, 4, 6, 6, 3, 1, 1, 1, 1, 0, 0),
]
# the literal reference call sequence swaps the stride and padding slots, so the kernels see stride = padding:
# a zero padding would be a zero stride (a division by zero in the reference's own CPU backend)
LITERAL = [
    (2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1),
    (2, 3, 9, 8, 4, 3, 3, 2, 2, 2, 2),
    (2, 2, 8, 8, 3, 3, 3, 2, 2, 1, 1),        # stride != padding: the kernels read pad 2, stride 1 with the layer's 4 x 4 output grid
]
# large enough for the tensor-core kernels (batched products with the weight shared by every batch)
TC = [
    (4, 16, 20, 20, 64, 3, 3, 1, 1, 1, 1),    # K = 144, P = 400, Cout = 64
    (3, 32, 12, 16, 72, 3, 3, 1, 1, 1, 1),    # ragged tiles: Cout = 72, P = 192
]


def _data(seed, dt, shape):
    B, C, Hh, W, Co, kh, kw = shape[:7]
    oh, ow, P, K = CC.geometry(*shape)
    rng = np.random.default_rng(seed)
    bound = 1.0 / np.sqrt(K)
    x = H.random_store(rng, dt, B * C * Hh * W, dist="normal")
    w = H.random_store(rng, dt, Co * K, lo=-bound, hi=bound)
    b = H.random_store(rng, dt, Co, lo=-bound, hi=bound)
    g = H.random_store(rng, dt, B * Co * P, dist="normal")
    return x, w, b, g


def _scales(shape):
    B, C, Hh, W, Co, kh, kw = shape[:7]
    oh, ow, P, K = CC.geometry(*shape)
    # magnitude of the sums each result is made of: out ~ sqrt(K) * |w| ~ 1; grad_x ~ sqrt(Co * kh * kw) * |w|; grad_w ~ sqrt(B * P)
    return {"out": 1.0, "grad_x": np.sqrt(Co * kh * kw / K), "grad_w": np.sqrt(B * P), "grad_bias": np.sqrt(B * P)}


def _rel(dt):
    return {"f32": 1e-4, "f64": 1e-10}.get(dt.name, 2e-2)


@pytest.mark.parametrize("dt", [D.F32, D.F64, D.BF16], ids=lambda d: d.name)
@pytest.mark.parametrize("shape", SMALL, ids=lambda s: "x".join(map(str, s)))
def test_oracle_direct_composition_is_a_convolution(oracle, dt, shape):
    from oracle import binding
    x, w, b, g = _data(11, dt, shape)
    binding.set_wide(True)
    try:
        got = CC.compose(oracle, dt, 1, shape, x, w, b, g)
    finally:
        binding.set_wide(False)
    ref = CC.direct_conv_f64(shape, D.decode(x, dt), D.decode(w, dt), D.decode(b, dt), D.decode(g, dt))
    sc = _scales(shape)
    for key in ("out", "grad_x", "grad_w", "grad_bias"):
        r = D.encode(ref[key], dt)
        H.assert_same("conv2d", dt, got[key], r, float_rel=_rel(dt), what=key, scale=sc[key])


def test_reference_call_sequence_differs_from_a_convolution_only_through_its_buffer_labels(oracle):
    """A 1x1 image under a padded 3x3 kernel has one output position (P = 1): the [B][K][P] and [B*P][K] labellings of the column buffer
    coincide, so the literal call sequence (mode 0) must give the convolution too."""
    dt = D.F32
    shape = (5, 4, 1, 1, 3, 3, 3, 1, 1, 1, 1)
    x, w, b, g = _data(12, dt, shape)
    got = CC.compose(oracle, dt, 0, shape, x, w, b, g)
    ref = CC.direct_conv_f64(shape, x, w, b, g)
    H.assert_same("conv2d", dt, got["out"], D.encode(ref["out"], dt), float_rel=1e-5, what="out", scale=1.0)
    # grad_x is not compared: the layer gives col2im num_els = B*C*H*W = 20, so only the first 20 of the 180 column
    # entries are read (crates/maidenx_cpu/src/nn/conv.rs:107,135)
    # the layer labels the [K, Cout] product as [Cout, C, kh, kw]: it is the transpose of the convolution's weight gradient
    gw = D.decode(got["grad_w"], dt).reshape(36, 3).T.reshape(-1)
    assert np.allclose(gw, ref["grad_w"], rtol=1e-5, atol=1e-5)


def _mode_cases():
    ident = lambda s: "x".join(map(str, s))  # noqa: E731
    return [pytest.param(0, s, id="reference-calls-" + ident(s)) for s in LITERAL + TC] + [pytest.param(1, s, id="direct-" + ident(s)) for s in SMALL + TC]


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [D.F32, D.BF16, D.F16, D.F64], ids=lambda d: d.name)
@pytest.mark.parametrize("mode,shape", _mode_cases())
def test_layer_matches_the_oracle_composed_the_same_way(oracle, cuda, dt, mode, shape):
    from oracle import binding
    x, w, b, g = _data(13, dt, shape)
    got = CC.run_layer(dt, mode, shape, x, w, b, g)
    binding.set_wide(True)
    try:
        ref = CC.compose(oracle, dt, mode, shape, x, w, b, g)
    finally:
        binding.set_wide(False)
    H.assert_same("conv2d_im2col", dt, got["cols"], ref["cols"], what="cols")  # a copy: bit-exact
    sc = _scales(shape)
    for key in ("out", "grad_x", "grad_w", "grad_bias"):
        # mode 0 multiplies re-labelled buffers: its sums have the same number of terms, so the same scales serve
        H.assert_same("conv2d", dt, got[key], ref[key], float_rel=_rel(dt), what=f"mode{mode}/{key}", scale=sc[key])


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [D.F32, D.BF16], ids=lambda d: d.name)
@pytest.mark.parametrize("shape", SMALL + TC, ids=lambda s: "x".join(map(str, s)))
def test_direct_layer_is_a_convolution(cuda, dt, shape):
    x, w, b, g = _data(14, dt, shape)
    got = CC.run_layer(dt, 1, shape, x, w, b, g)
    ref = CC.direct_conv_f64(shape, D.decode(x, dt), D.decode(w, dt), D.decode(b, dt), D.decode(g, dt))
    sc = _scales(shape)
    for key in ("out", "grad_x", "grad_w", "grad_bias"):
        H.assert_same("conv2d", dt, got[key], D.encode(ref[key], dt), float_rel=_rel(dt), what=key, scale=sc[key])


@pytest.mark.gpu
def test_literal_call_sequence_is_refused_when_the_swapped_slots_would_mean_a_zero_stride(cuda):
    import ctypes
    from maidenx_b200 import _lib
    lib = _lib.load()
    conv = _lib.MxConv2d(1, 1, 4, 4, 1, 1, 1, 1, 1, 0, 0)
    fwd, _ = _lib.conv2d("f32")
    lib.mx_clear_error()
    fwd(ctypes.byref(conv), 0, 1, 1, None, 1, 1, 1)  # refused before any pointer is touched
    assert lib.mx_last_error() == 3
    lib.mx_clear_error()


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [D.BF16, D.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("shape", [(8, 32, 24, 24, 128, 3, 3, 1, 1, 1, 1), (5, 16, 20, 24, 200, 3, 3, 1, 1, 1, 1)], ids=lambda s: "x".join(map(str, s)))
def test_bias_in_the_product_epilogue_equals_the_separate_add(cuda, dt, shape):
    """Direct form, 16-bit types, shapes the tensor-core kernel takes: the per-channel bias rides in the batched
    product's epilogue (one bias element per output row).  Bit for bit what cuda_matmul followed by cuda_add_inplace
    gives (the op-by-op composition on the same backend), with ragged row tiles (200 channels) as well."""
    x, w, b, g = _data(15, dt, shape)
    got = CC.run_layer(dt, 1, shape, x, w, b, g)
    ref = CC.compose(cuda, dt, 1, shape, x, w, b, g)
    assert np.array_equal(got["out"], ref["out"])
    for key in ("grad_x", "grad_w", "grad_bias"):
        assert np.array_equal(got[key], ref[key]), key
