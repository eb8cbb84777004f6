"""Parity of conv2d im2col / col2im against the CPU oracle, through the C ABI, on a B200.
Both are copies or short fixed-order sums in the element type, so the bar is bit-exact for
all four float dtypes.  Nothing in the reference pins these values (its Conv2d tests check
shapes only), so the oracle's restatement of crates/maidenx_cpu/src/nn/conv.rs is the
definition.  col2im is exercised both with num_els = the full col length and with the value
the reference's Conv2d passes, B*C*H*W (crates/maidenx_nn/src/layers/conv.rs:393), which
makes every col entry at or beyond it invisible.
"""
import numpy as np
import pytest

import harness as H
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu


def cases():
    """(name, B, C, H, W, kh, kw, ph, pw, sh, sw)"""
    return [
        ("3x3-s1-p1", 2, 3, 8, 8, 3, 3, 1, 1, 1, 1),
        ("3x3-s1-p1-vec", 2, 4, 16, 16, 3, 3, 1, 1, 1, 1),
        ("5x5-s2-p2", 1, 2, 13, 11, 5, 5, 2, 2, 2, 2),
        ("2x3-mixed", 2, 2, 9, 10, 2, 3, 0, 1, 1, 2),
        ("1x1", 3, 5, 7, 7, 1, 1, 0, 0, 1, 1),
        ("no-pad", 1, 3, 12, 12, 3, 3, 0, 0, 1, 1),
        ("s3", 1, 1, 20, 17, 3, 3, 1, 1, 3, 3),
        ("big-plane", 1, 2, 56, 56, 3, 3, 1, 1, 1, 1),
        # stride-1 vector fast paths: widths that are multiples of the 16-byte vector, kw in {1,3,5,7}
        ("5x5-s1-p2-vec", 2, 2, 16, 24, 5, 5, 2, 2, 1, 1),
        ("7x7-s1-p3-vec", 1, 1, 16, 16, 7, 7, 3, 3, 1, 1),
        ("1x1-vec", 2, 3, 8, 16, 1, 1, 0, 0, 1, 1),
        ("1x3-vec", 1, 2, 9, 16, 1, 3, 0, 1, 1, 1),
        ("3x1-vec", 1, 2, 9, 16, 3, 1, 1, 0, 1, 1),
        ("3x3-s1-p0", 1, 2, 10, 10, 3, 3, 0, 0, 1, 1),
        ("3x3-s1-p1-tall", 3, 2, 40, 8, 3, 3, 1, 1, 1, 1),
    ]


def _geom(c):
    _, B, C, Hh, W, kh, kw, ph, pw, sh, sw = c
    oh = (Hh + 2 * ph - kh) // sh + 1
    ow = (W + 2 * pw - kw) // sw + 1
    return B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw


@pytest.mark.parametrize("dt", D.FLOATS, ids=lambda d: d.name)
def test_im2col(oracle, cuda, dt):
    rng = np.random.default_rng(31)
    for c in cases():
        B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw = _geom(c)
        meta = H.conv_metadata(B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw)
        x = H.random_store(rng, dt, B * C * Hh * W, dist="normal")
        n = B * C * kh * kw * oh * ow
        ref = H.run_im2col(oracle, dt, meta, n, x)
        got = H.run_im2col(cuda, dt, meta, n, x)
        H.assert_same("conv2d_im2col", dt, got, ref, what=c[0])


@pytest.mark.parametrize("dt", D.FLOATS, ids=lambda d: d.name)
def test_col2im(oracle, cuda, dt):
    rng = np.random.default_rng(32)
    for c in cases():
        B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw = _geom(c)
        meta = H.conv_metadata(B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw)
        ncol = B * C * kh * kw * oh * ow
        col = H.random_store(rng, dt, ncol, dist="normal")
        out_len = B * C * Hh * W
        for num_els in (ncol, min(ncol, out_len)):
            ref = H.run_col2im(oracle, dt, meta, num_els, col, out_len)
            got = H.run_col2im(cuda, dt, meta, num_els, col, out_len)
            H.assert_same("conv2d_col2im", dt, got, ref, what=f"{c[0]} num_els={num_els}")


def test_im2col_col2im_adjoint(cuda):
    """<im2col(x), y> == <x, col2im(y)> (the two are adjoint linear maps): a size-independent
    property, checked here in f64."""
    rng = np.random.default_rng(33)
    dt = D.F64
    B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw = _geom(("", 2, 3, 10, 9, 3, 3, 1, 1, 2, 1))
    meta = H.conv_metadata(B, C, Hh, W, kh, kw, oh, ow, ph, pw, sh, sw)
    ncol = B * C * kh * kw * oh * ow
    x = rng.standard_normal(B * C * Hh * W)
    y = rng.standard_normal(ncol)
    cx = H.run_im2col(cuda, dt, meta, ncol, x)
    ty = H.run_col2im(cuda, dt, meta, ncol, y, x.size)
    assert np.isclose(np.dot(cx, y), np.dot(x, ty), rtol=1e-12)
