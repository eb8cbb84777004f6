"""CPU-only checks of the training-step logic: the oracle-composed MLP against a numpy model,
and the data-parallel rule (shard the batch, all-reduce-average the gradients) on two gloo
ranks against a single process on the whole batch."""
import os
import socket

import numpy as np
import pytest

from maidenx_b200 import dtypes as D


def _model(L, Dm, seed):
    rng = np.random.default_rng(seed)
    bound = 1.0 / np.sqrt(Dm)
    W = [rng.uniform(-bound, bound, Dm * Dm).astype(np.float32) for _ in range(L)]
    b = [rng.uniform(-bound, bound, 1).astype(np.float32) for _ in range(L)]
    return W, b


def _numpy_grads(W, b, x, y, L, Dm, B):
    gelu = lambda v: 0.5 * v * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))

    def dgelu(v):
        s, c = 0.7978845608028654, 0.044715
        t = np.tanh(s * (v + c * v ** 3))
        return 0.5 * (1 + t) + 0.5 * v * (1 - t * t) * s * (1 + 3 * c * v * v)

    a, us = [x.reshape(B, Dm).astype(np.float64)], []
    for l in range(L):
        u = a[-1] @ W[l].reshape(Dm, Dm).astype(np.float64).T + float(b[l][0])
        us.append(u)
        a.append(gelu(u) if l < L - 1 else u)
    diff = us[-1] - y.reshape(B, Dm)
    loss = np.mean(diff ** 2)
    du = 2 * diff / diff.size
    gW, gb = [None] * L, [None] * L
    for l in reversed(range(L)):
        if l < L - 1:
            du = da * dgelu(us[l])
        gW[l], gb[l] = du.T @ a[l], du.sum()
        da = du @ W[l].reshape(Dm, Dm)
    return loss, gW, gb


def test_oracle_mlp_matches_numpy_model():
    from oracle.mlp_reference import CpuMlp
    L, Dm, B = 3, 16, 24
    W, b = _model(L, Dm, 1)
    rng = np.random.default_rng(2)
    x, y = rng.standard_normal(B * Dm).astype(np.float32), rng.standard_normal(B * Dm).astype(np.float32)
    m = CpuMlp(L, Dm, B, "f32", [w.copy() for w in W], [v.copy() for v in b])
    loss, gW, gb = m.gradients(x, y)
    rl, rW, rb = _numpy_grads(W, b, x, y, L, Dm, B)
    assert np.isclose(loss[0], rl, rtol=1e-5)
    for l in range(L):
        assert np.allclose(gW[l].reshape(Dm, Dm), rW[l], rtol=1e-4, atol=1e-7)
        assert np.isclose(gb[l][0], rb[l], rtol=1e-4, atol=1e-7)
    m.apply(gW, gb, 0.1)
    assert np.allclose(m.W[0], W[0] - 0.1 * gW[0], rtol=1e-6)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _dp_worker(rank, world, port, L, Dm, B, q):
    import torch
    import torch.distributed as dist
    from oracle.mlp_reference import CpuMlp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    W, b = _model(L, Dm, 1)                      # identical weights on every rank
    rng = np.random.default_rng(2)
    x, y = rng.standard_normal(B * Dm).astype(np.float32), rng.standard_normal(B * Dm).astype(np.float32)
    local = B // world
    xs, ys = x[rank * local * Dm:(rank + 1) * local * Dm].copy(), y[rank * local * Dm:(rank + 1) * local * Dm].copy()
    m = CpuMlp(L, Dm, local, "f32", W, b)
    _, gW, gb = m.gradients(xs, ys)
    for l in reversed(range(L)):                 # one bucket per layer, averaged
        for g in (gW[l], gb[l]):
            t = torch.from_numpy(g)
            dist.all_reduce(t)
            t /= world
    m.apply(gW, gb, 0.1)
    if rank == 0:
        q.put([w.copy() for w in m.W])
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_data_parallel_step_equals_single_process_step():
    import torch.multiprocessing as mp
    from oracle.mlp_reference import CpuMlp
    L, Dm, B, world = 2, 16, 16, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dp_worker, args=(r, world, port, L, Dm, B, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    W, b = _model(L, Dm, 1)
    rng = np.random.default_rng(2)
    x, y = rng.standard_normal(B * Dm).astype(np.float32), rng.standard_normal(B * Dm).astype(np.float32)
    m = CpuMlp(L, Dm, B, "f32", W, b)
    m.step(x, y, 0.1)
    for l in range(L):
        assert np.allclose(got[l], m.W[l], rtol=1e-5, atol=1e-7)
