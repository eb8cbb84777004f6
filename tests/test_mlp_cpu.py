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


def _sharded_worker(rank, world, port, L, Dm, B, q):
    """The exchange the CUDA data-parallel engine performs (csrc/dp_sync.cu), restated over gloo: every rank sums,
    in rank order, only ITS 1/world shard of each layer's gradients, updates that shard of the weights, and the
    shards are gathered back so that all ranks hold the full new weights."""
    import torch
    import torch.distributed as dist
    from oracle.mlp_reference import CpuMlp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    W, b = _model(L, Dm, 1)
    rng = np.random.default_rng(2)
    x, y = rng.standard_normal(B * Dm).astype(np.float32), rng.standard_normal(B * Dm).astype(np.float32)
    local = B // world
    xs, ys = x[rank * local * Dm:(rank + 1) * local * Dm].copy(), y[rank * local * Dm:(rank + 1) * local * Dm].copy()
    m = CpuMlp(L, Dm, local, "f32", W, b)
    _, gW, gb = m.gradients(xs, ys)
    lr, scale = np.float32(0.1), np.float32(1.0 / world)
    n = Dm * Dm
    shard = n // world
    lo, hi = rank * shard, (rank + 1) * shard
    for l in reversed(range(L)):
        # "peer loads": my shard of every rank's gradient, summed in rank order
        pieces = [torch.empty(shard, dtype=torch.float32) for _ in range(world)]
        for owner in range(world):                       # rank `owner` collects shard `owner` from everyone
            mine = torch.from_numpy(gW[l][owner * shard:(owner + 1) * shard].copy())
            dist.gather(mine, pieces if rank == owner else None, dst=owner)
        acc = np.zeros(shard, dtype=np.float32)
        for p in range(world):
            acc = acc + pieces[p].numpy()
        new_shard = m.W[l][lo:hi] - (lr * scale) * acc   # the update touches 1/world of the weights
        # "peer stores": every rank receives every shard
        out = [torch.empty(shard, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(out, torch.from_numpy(new_shard.astype(np.float32)))
        m.W[l] = np.concatenate([t.numpy() for t in out])
        # the scalar bias: every rank adds all ranks' gradients in rank order
        gbs = [torch.empty(1, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gbs, torch.from_numpy(gb[l].copy()))
        s = np.float32(0)
        for t in gbs:
            s = np.float32(s + t.numpy()[0])
        m.b[l] = (m.b[l] - (lr * scale) * s).astype(np.float32)
    q.put((rank, [w.copy() for w in m.W], [v.copy() for v in m.b]))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_reduce_update_gather_equals_single_process_step():
    import torch.multiprocessing as mp
    from oracle.mlp_reference import CpuMlp
    L, Dm, B, world = 2, 16, 16, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_worker, args=(r, world, port, L, Dm, B, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict((r, (w, bb)) for r, w, bb in (q.get(timeout=120) for _ in range(world)))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # every rank ends with bit-identical parameters ...
    for l in range(L):
        assert np.array_equal(results[0][0][l], results[1][0][l]) and np.array_equal(results[0][1][l], results[1][1][l])
    # ... and they are those of one process training on the whole batch
    W, b = _model(L, Dm, 1)
    rng = np.random.default_rng(2)
    x, y = rng.standard_normal(B * Dm).astype(np.float32), rng.standard_normal(B * Dm).astype(np.float32)
    m = CpuMlp(L, Dm, B, "f32", W, b)
    m.step(x, y, 0.1)
    for l in range(L):
        assert np.allclose(results[0][0][l], m.W[l], rtol=1e-5, atol=1e-7)
        assert np.allclose(results[0][1][l], m.b[l], rtol=1e-5, atol=1e-7)
