"""The reference's README training example with every tensor resident on the device.

Linear(3 -> 1, bias) + MSE + SGD(lr = 0.01) in f32 on a 10000 x 3 batch (README.md:59-101, examples/device/cuda.rs of
the reference), issued op by op in the order the reference's eager autograd issues them:

  forward     x.matmul(W^T view) then add(bias)                       crates/maidenx_nn/src/layers/linear.rs:60-81
  loss        sub, pow(2), sum of every dim, div_scalar(n)            crates/maidenx_nn/src/losses/mse.rs:21-29
  backward    1/n, pow' (mul_scalar 2 of pow 1), mul; the bias gradient is the sum_to_shape fold of the
              broadcast add; dW = dpred^T . x as a strided matmul
  SGD.step    param.sub_(grad.mul_scalar(lr))                         crates/maidenx_nn/src/optimizers/sgd.rs:17-26

`train(engine, steps)` is written against a small engine interface so that the same sequence runs on the CUDA library
(`CudaEngine`: every op output is a cuda_malloc'ed buffer, every call uploads its metadata block, calls the op and
frees the block, exactly as maidenx_core does; intermediates are freed when the step no longer needs them) and on any
other backend that offers the same three methods.  17 op calls per step; the loss is read back every `read_every` steps
(the example prints it every 100 epochs).
"""
from __future__ import annotations

import ctypes

import numpy as np

N, K, LR = 10000, 3, 0.01
SZ = ctypes.c_size_t
OPS_PER_STEP = 17


def dataset():
    i = np.arange(N) % 100
    x = np.stack([i / 100.0, (i + 1) / 100.0, (i + 2) / 100.0], axis=1).astype(np.float32)
    y = ((i * 10) / 1000.0).astype(np.float32).reshape(N, 1)
    return x, y


def initial_parameters():
    """The reference draws them from an unseeded generator; here they are fixed."""
    return np.array([0.3, -0.2, 0.1], dtype=np.float32), np.array([0.05], dtype=np.float32)


class CudaEngine:
    """Device buffers from cuda_malloc, ops through the reference's dispatch pattern (maidenx_b200.device.dispatch)."""
    name = "cuda"

    def __init__(self):
        from . import device
        self.device = device

    def upload(self, arr):
        return self.device.CudaBuffer.from_host(np.ascontiguousarray(arr, dtype=np.float32))

    def empty(self, count):
        return self.device.CudaBuffer(4 * max(count, 1))

    def free(self, buf):
        buf.free()

    def ptr(self, buf):
        return buf.ptr

    def call(self, op, metadata, *args):
        self.device.dispatch(op, "f32", metadata, *args, check=False)

    def read(self, buf, count):
        return buf.to_host(np.float32, count)


def _f32(v):
    return ctypes.c_float(v)


def train(engine, steps, read_every=100):
    """Runs `steps` SGD steps; returns (losses read back, W, b)."""
    e = engine
    x, y = dataset()
    W0, b0 = initial_parameters()
    xs, ys, W, b = e.upload(x.ravel()), e.upload(y.ravel()), e.upload(W0), e.upload(b0)
    one = e.upload(np.ones(1, np.float32))
    p = e.ptr
    losses = []
    for step in range(steps):
        tmp = []

        def new(count):
            buf = e.empty(count)
            tmp.append(buf)
            return buf

        # forward: [N, 3] . W^T (W stored [1, 3]; its transposed view has shape [3, 1], strides [1, 3]), + bias
        z = new(N)
        e.call("matmul", [2, 2, 2, N, 1, N, K, K, 1, K, 1, 1, K, 0, 0], SZ(N), "META", p(xs), p(W), p(z))
        pred = new(N)
        e.call("add", [N, 1, 1, 1, 0, 0, 0, 0], SZ(N), SZ(2), "META", p(z), p(b), p(pred))
        # loss
        diff = new(N)
        e.call("sub", [N, 1, 1, 1, 1, 1, 0, 0], SZ(N), SZ(2), "META", p(pred), p(ys), p(diff))
        sq = new(N)
        e.call("pow", [N, 1, 1, 1, 0], SZ(N), SZ(2), "META", p(diff), _f32(2.0), p(sq))
        s1 = new(N)
        e.call("sum", [N, 1, 1, 1, 1, 1, 0], SZ(N), SZ(2), SZ(1), "META", p(sq), p(s1))            # dim 1 (length 1)
        total = new(1)
        e.call("sum", [N, 1, N, 1, 0], SZ(N), SZ(1), SZ(1), "META", p(s1), p(total))               # dim 0
        loss = new(1)
        e.call("div_scalar", [1, 1, 0], SZ(1), SZ(1), "META", p(total), _f32(float(N)), p(loss))
        # backward of the loss
        g = new(1)
        e.call("div_scalar", [1, 1, 0], SZ(1), SZ(1), "META", p(one), _f32(float(N)), p(g))
        p1 = new(N)
        e.call("pow", [N, 1, 1, 1, 0], SZ(N), SZ(2), "META", p(diff), _f32(1.0), p(p1))
        two_diff = new(N)
        e.call("mul_scalar", [N, 1, 1, 1, 0], SZ(N), SZ(2), "META", p(p1), _f32(2.0), p(two_diff))
        dpred = new(N)
        e.call("mul", [N, 1, 1, 1, 0, 0, 0, 0], SZ(N), SZ(2), "META", p(two_diff), p(g), p(dpred))
        db = new(1)
        e.call("sum_to_shape", [N, 1, 1, 1, 1, 1, 0], SZ(N), SZ(2), "META", p(dpred), p(db))       # fold of the broadcast add
        dW = new(K)
        e.call("matmul", [2, 2, 2, 1, K, 1, N, N, K, 1, 1, K, 1, 0, 0], SZ(K), "META", p(dpred), p(xs), p(dW))  # dpred^T [1, N] . x [N, 3]
        # SGD
        sW, sb = new(K), new(1)
        e.call("mul_scalar", [K, 1, 0], SZ(K), SZ(1), "META", p(dW), _f32(LR), p(sW))
        e.call("sub_inplace", [K, 1, 1, 0, 0], SZ(K), SZ(1), "META", p(W), p(sW))
        e.call("mul_scalar", [1, 1, 0], SZ(1), SZ(1), "META", p(db), _f32(LR), p(sb))
        e.call("sub_inplace", [1, 1, 1, 0, 0], SZ(1), SZ(1), "META", p(b), p(sb))
        if (step + 1) % read_every == 0 or step == steps - 1:
            losses.append(float(e.read(loss, 1)[0]))
        for buf in tmp:
            e.free(buf)
    Wf, bf = e.read(W, K), e.read(b, 1)
    for buf in (xs, ys, W, b, one):
        e.free(buf)
    return losses, Wf, bf
