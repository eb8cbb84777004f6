"""TEST INFRASTRUCTURE ONLY: the MLP training step composed from CPU-oracle ops in the order the
reference's eager autograd issues them, used as the checker in tests and as the timed CPU arm.

Call sequence (citations are paths inside the reference project):
  Linear.forward   x.matmul(W.transpose(-1,-2)) then add(bias)          crates/maidenx_nn/src/layers/linear.rs:60-81
  GELU             gelu forward; backward = the elementwise closure      crates/maidenx_tensor/src/ops/unary.rs:298-352
  MSELoss          sub, pow(2), sum over each dim, div_scalar            crates/maidenx_nn/src/losses/mse.rs:21-29
  backward         div_scalar^-1, broadcast, pow' (mul_scalar, pow(1), mul), sub', add' (sum_to_shape),
                   matmul_backward with both gradients                   crates/maidenx_tensor/src/ops/matmul.rs:63-111
  SGD.step         grad.mul_scalar(lr) then param.sub_(...)               crates/maidenx_nn/src/optimizers/sgd.rs:17-26
Two deliberate differences from a literal replay, both stated where they occur: the weight
gradient and input gradient are the mathematically correct products (see `correct_backward`),
and scalars that the reference promotes to F32 stay in the working dtype.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import binding

SZ = ctypes.c_size_t


def _np(dt):
    return {"bf16": np.uint16, "f16": np.float16, "f32": np.float32, "f64": np.float64}[dt]


def _enc(values, dt):
    from maidenx_b200 import dtypes as D
    return D.encode(values, D.BY_NAME[dt])


def _scalar(v, dt):
    from maidenx_b200 import dtypes as D
    return D.scalar_arg(v, D.BY_NAME[dt])


class Ops:
    """Thin positional wrappers over the oracle's C entry points on numpy buffers."""

    def __init__(self, dt: str):
        binding.load()
        self.dt = dt
        self.npdt = _np(dt)

    def binary(self, op, a, b, dims, sa, sb):
        n = int(np.prod(dims)) if dims else 1
        out = np.empty(n, self.npdt)
        meta = np.asarray(list(dims) + list(sa) + list(sb) + [0, 0], dtype=np.uint64)
        binding.op(op, self.dt)(SZ(n), SZ(len(dims)), meta.ctypes.data, a.ctypes.data, b.ctypes.data, out.ctypes.data)
        return out

    def unary(self, op, a, n, scalar=None):
        out = np.empty(n, self.npdt)
        meta = np.asarray([n, 1, 0], dtype=np.uint64)
        if scalar is None:
            binding.op(op, self.dt)(SZ(n), SZ(1), meta.ctypes.data, a.ctypes.data, out.ctypes.data)
        else:
            binding.op(op, self.dt)(SZ(n), SZ(1), meta.ctypes.data, a.ctypes.data, _scalar(scalar, self.dt), out.ctypes.data)
        return out

    def inplace(self, op, a, b, n):
        meta = np.asarray([n, 1, 1, 0, 0], dtype=np.uint64)
        binding.op(op, self.dt)(SZ(n), SZ(1), meta.ctypes.data, a.ctypes.data, b.ctypes.data)

    def sum_dim(self, a, dims, dim):
        st = []
        acc = 1
        for d in reversed(dims):
            st.insert(0, acc)
            acc *= d
        n = int(np.prod(dims))
        out = np.empty(max(n // dims[dim], 1), self.npdt)
        meta = np.asarray(list(dims) + st + [dims[dim], st[dim], 0], dtype=np.uint64)
        binding.op("sum", self.dt)(SZ(n), SZ(len(dims)), SZ(1), meta.ctypes.data, a.ctypes.data, out.ctypes.data)
        return out

    def matmul(self, a, b, out_shape, a_shape, b_shape, a_st, b_st):
        n = int(np.prod(out_shape))
        out = np.empty(n, self.npdt)
        meta = np.asarray([2, 2, 2] + list(out_shape) + list(a_shape) + list(b_shape) + list(a_st) + list(b_st) + [0, 0], dtype=np.uint64)
        binding.op("matmul", self.dt)(SZ(n), meta.ctypes.data, a.ctypes.data, b.ctypes.data, out.ctypes.data)
        return out


class CpuMlp:
    """L x [Linear(D -> D) + scalar bias, GELU between layers], MSE, SGD on the CPU oracle."""

    def __init__(self, layers, dim, batch, dt, weights, biases):
        self.L, self.D, self.B, self.dt = layers, dim, batch, dt
        self.ops = Ops(dt)
        self.W = [np.ascontiguousarray(w) for w in weights]  # stored bits, [D*D]
        self.b = [np.ascontiguousarray(b) for b in biases]   # stored bits, [1]

    def gelu_backward(self, u, grad, n):
        """The reference's closure, op by op (unary.rs:324-346)."""
        o = self.ops
        s, c = 0.7978845608028654, 0.044715
        flat, one = [n], [1]
        x2 = o.binary("mul", u, u, flat, one, one)
        x3 = o.binary("mul", x2, u, flat, one, one)
        targ = o.unary("mul_scalar", o.binary("add", u, o.unary("mul_scalar", x3, n, c), flat, one, one), n, s)
        th = o.unary("tanh", targ, n)
        sech2 = o.unary("add_scalar", o.unary("mul_scalar", o.binary("mul", th, th, flat, one, one), n, -1.0), n, 1.0)
        inner = o.unary("mul_scalar", o.unary("add_scalar", o.unary("mul_scalar", x2, n, 3.0 * c), n, 1.0), n, s)
        term1 = o.unary("mul_scalar", o.unary("add_scalar", th, n, 1.0), n, 0.5)
        term2 = o.unary("mul_scalar", o.binary("mul", o.binary("mul", u, sech2, flat, one, one), inner, flat, one, one), n, 0.5)
        return o.binary("mul", grad, o.binary("add", term1, term2, flat, one, one), flat, one, one)

    def gradients(self, x, y):
        """Forward + backward; returns (loss, [dW], [db]) as stored bits, weights untouched."""
        o, L, D, B = self.ops, self.L, self.D, self.B
        n = B * D
        acts, us = [x], []
        for l in range(L):
            z = o.matmul(acts[-1], self.W[l], [B, D], [B, D], [D, D], [D, 1], [1, D])  # B = W^T view
            u = o.binary("add", z, self.b[l], [B, D], [D, 1], [0, 0])
            us.append(u)
            acts.append(o.unary("gelu", u, n) if l < L - 1 else u)
        diff = o.binary("sub", us[-1], y, [n], [1], [1])
        sq = o.unary("pow", diff, n, 2.0)
        total = o.sum_dim(o.sum_dim(sq, [B, D], 1), [B], 0)
        loss = o.unary("div_scalar", total, 1, float(n))
        # backward of the loss: d/dpred = 2 * diff / n
        g = o.unary("div_scalar", _enc(np.ones(1), self.dt), 1, float(n))
        du = o.binary("mul", o.unary("mul_scalar", o.unary("pow", diff, n, 1.0), n, 2.0), g, [n], [1], [0])
        gWs, gbs = [None] * L, [None] * L
        for l in reversed(range(L)):
            if l < L - 1:
                du = self.gelu_backward(us[l], da, n)
            gbs[l] = o.sum_dim(o.sum_dim(du, [B, D], 1), [B], 0)
            # correct_backward: dW = du^T . a_prev and da = du . W as two strided matmuls, the form the
            # reference's graph mode uses (crates/maidenx_tensor_v2/src/ops/_try_matmul.rs:98-140)
            gWs[l] = o.matmul(du, acts[l], [D, D], [D, B], [B, D], [1, D], [D, 1])
            if l > 0:
                da = o.matmul(du, self.W[l], [B, D], [B, D], [D, D], [D, 1], [D, 1])
        self.last_output = us[-1]
        return loss, gWs, gbs

    def apply(self, gWs, gbs, lr):
        """SGD.step: param.sub_(grad.mul_scalar(lr))."""
        o, D = self.ops, self.D
        for l in range(self.L):
            o.inplace("sub_inplace", self.W[l], o.unary("mul_scalar", gWs[l], D * D, lr), D * D)
            o.inplace("sub_inplace", self.b[l], o.unary("mul_scalar", gbs[l], 1, lr), 1)

    def step(self, x, y, lr):
        loss, gWs, gbs = self.gradients(x, y)
        self.apply(gWs, gbs, lr)
        return loss
