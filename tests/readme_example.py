"""The reference's README training example - Linear(3 -> 1, bias) + MSE + SGD(lr = 0.01) in f32 on a
10000 x 3 batch - composed from single op calls in the order the reference's eager autograd issues
them, on whichever backend (CPU oracle or the CUDA library) it is given.

  input row i = [(i % 100) / 100, (i % 100 + 1) / 100, (i % 100 + 2) / 100], target ((i % 100) * 10) / 1000
  forward     x.matmul(W^T view) then add(bias)                       crates/maidenx_nn/src/layers/linear.rs:60-81
  loss        sub, pow(2), sum of every dim, div_scalar(n)            crates/maidenx_nn/src/losses/mse.rs:21-29
  backward    1/n, pow' (mul_scalar 2 of pow 1), mul; the bias gradient is the sum_to_shape fold of the
              broadcast add; dW = dpred^T . x as a strided matmul
  SGD.step    param.sub_(grad.mul_scalar(lr))                         crates/maidenx_nn/src/optimizers/sgd.rs:17-26
The reference draws the initial weights from an unseeded generator; here they are fixed.
"""
import numpy as np

import harness as H
from maidenx_b200 import dtypes as D

N, K = 10000, 3
LR = 0.01


def dataset():
    i = np.arange(N) % 100
    x = np.stack([i / 100.0, (i + 1) / 100.0, (i + 2) / 100.0], axis=1).astype(np.float32)
    y = ((i * 10) / 1000.0).astype(np.float32).reshape(N, 1)
    return x, y


def initial_parameters():
    return np.array([0.3, -0.2, 0.1], dtype=np.float32), np.array([0.05], dtype=np.float32)


def train(be, steps):
    """Returns (losses, W, b) after `steps` SGD steps, every tensor op going through backend `be`."""
    dt = D.F32
    x, y = dataset()
    xs, ys = x.ravel().copy(), y.ravel().copy()
    W, b = initial_parameters()
    losses = []
    for _ in range(steps):
        # forward: [N, 3] . W^T, W stored as [1, 3] -> its transposed view has shape [3, 1], strides [1, 3]
        meta = H.matmul_metadata([N, 1], [N, K], [K, 1], [K, 1], [1, K], 0, 0)
        z = H.run_matmul(be, dt, meta, N, xs, W)
        pred = H.run_binary(be, "add", dt, [N, 1], [1, 1], [0, 0], 0, 0, z, b)
        # loss
        diff = H.run_binary(be, "sub", dt, [N, 1], [1, 1], [1, 1], 0, 0, pred, ys)
        sq = H.run_unary(be, "pow", dt, [N, 1], [1, 1], 0, diff, scalar=2.0)
        s1 = H.run_reduce(be, "sum", dt, [N, 1], [1, 1], [1], [1], 0, sq)           # dim 1 (length 1)
        total = H.run_reduce(be, "sum", dt, [N], [1], [N], [1], 0, s1)             # dim 0
        loss = H.run_unary(be, "div_scalar", dt, [1], [1], 0, total, scalar=float(N))
        losses.append(float(loss[0]))
        # backward of the loss
        g = H.run_unary(be, "div_scalar", dt, [1], [1], 0, np.ones(1, dtype=np.float32), scalar=float(N))
        two_diff = H.run_unary(be, "mul_scalar", dt, [N, 1], [1, 1], 0, H.run_unary(be, "pow", dt, [N, 1], [1, 1], 0, diff, scalar=1.0), scalar=2.0)
        dpred = H.run_binary(be, "mul", dt, [N, 1], [1, 1], [0, 0], 0, 0, two_diff, g)
        # bias gradient: the broadcast add folds its gradient back to the bias shape
        db = H.run_sum_to_shape(be, dt, [N, 1], [1, 1], [1, 1], 0, dpred)
        # weight gradient [1, 3] = dpred^T [1, N] (a view of dpred with strides [1, 1]) . x [N, 3]
        meta = H.matmul_metadata([1, K], [1, N], [N, K], [1, 1], [K, 1], 0, 0)
        dW = H.run_matmul(be, dt, meta, K, dpred, xs)
        # SGD
        W = H.run_binary_inplace(be, "sub_inplace", dt, [K], [1], [1], 0, 0, W, H.run_unary(be, "mul_scalar", dt, [K], [1], 0, dW, scalar=LR))
        b = H.run_binary_inplace(be, "sub_inplace", dt, [1], [1], [1], 0, 0, b, H.run_unary(be, "mul_scalar", dt, [1], [1], 0, db, scalar=LR))
    return losses, W, b


def train_numpy(steps):
    """The same model in float64, closed-form gradients."""
    x, y = dataset()
    x, y = x.astype(np.float64), y.astype(np.float64)
    W, b = (p.astype(np.float64) for p in initial_parameters())
    losses = []
    for _ in range(steps):
        diff = x @ W.reshape(K, 1) + b - y
        losses.append(float(np.mean(diff ** 2)))
        dpred = 2.0 * diff / N
        W = W - LR * (dpred.T @ x).ravel()
        b = b - LR * dpred.sum()
    return losses, W, b
