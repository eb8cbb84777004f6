"""The MLP training step (csrc/mlp.cu + fused kernels) checked on a B200:
  * the fused elementwise passes against the chain of single-op C-ABI calls they stand for,
    which in turn is checked against the CPU oracle elsewhere;
  * one whole step (forward, loss, every gradient, SGD update) against an f64 numpy evaluation
    of the same model from the same seeded weights, within bf16 tolerance;
  * the loss goes down over a few steps.
Sizes are small enough for numpy but large enough (M*N*K >= 2^24) that every matrix product
runs on the tensor-core path.
"""
import ctypes

import numpy as np
import pytest

import harness as H
from maidenx_b200 import _lib, device
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu
SZ = ctypes.c_size_t


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def init_uniform(seed, n, bound):
    """The engine's counter-based initialiser (mlp.cu: splitmix64 of seed * 0x100000001B3 + i)."""
    with np.errstate(over="ignore"):
        i = np.arange(n, dtype=np.uint64)
        r = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + i)
    u = (r >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return (np.float32(2.0) * u - np.float32(1.0)) * np.float32(bound)


def gelu64(x):
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def gelu_grad64(x):
    s, c = 0.7978845608028654, 0.044715
    t = np.tanh(s * (x + c * x ** 3))
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * s * (1 + 3 * c * x * x)


def bf(x):
    """Round an array to bf16 and back (f64 result)."""
    return D.decode(D.encode(np.asarray(x, dtype=np.float32), D.BF16), D.BF16)


def test_fused_passes_match_the_single_op_chain(cuda):
    lib = _lib.load()
    rng = np.random.default_rng(0)
    n = 40_000
    dt = D.BF16
    z = H.random_store(rng, dt, n, dist="normal")
    b = D.encode([0.37], dt)
    # chain: add with a broadcast scalar rhs, then gelu
    u_ref = H.run_binary(cuda, "add", dt, [n], [1], [0], 0, 0, z, b)
    a_ref = H.run_unary(cuda, "gelu", dt, [n], [1], 0, u_ref)
    zb, bb = device.CudaBuffer.from_host(z), device.CudaBuffer.from_host(np.resize(b, 128))
    ub, ab = device.CudaBuffer(n * 2), device.CudaBuffer(n * 2)
    lib.mx_bias_gelu_bf16(n, zb.ptr, bb.ptr, ub.ptr, ab.ptr)
    device.synchronize()
    assert np.array_equal(ub.to_host(np.uint16, n), u_ref) and np.array_equal(ab.to_host(np.uint16, n), a_ref)
    # gelu backward against f64
    dy = H.random_store(rng, dt, n, dist="normal")
    dyb, dub = device.CudaBuffer.from_host(dy), device.CudaBuffer(n * 2)
    lib.mx_gelu_backward_bf16(n, dyb.ptr, ub.ptr, dub.ptr)
    device.synchronize()
    want = D.decode(dy, dt) * gelu_grad64(D.decode(u_ref, dt))
    got = D.decode(dub.to_host(np.uint16, n), dt)
    assert np.all(np.abs(got - want) <= 1e-2 * np.maximum(np.abs(want), np.abs(D.decode(dy, dt)) * 1e-1))
    # mse: loss and gradient
    p, t = H.random_store(rng, dt, n, dist="normal"), H.random_store(rng, dt, n, dist="normal")
    pb, tb, gb, lb = device.CudaBuffer.from_host(p), device.CudaBuffer.from_host(t), device.CudaBuffer(n * 2), device.CudaBuffer(256)
    lib.mx_mse_loss_grad_bf16(n, pb.ptr, tb.ptr, gb.ptr, lb.ptr)
    device.synchronize()
    diff = bf(D.decode(p, dt) - D.decode(t, dt))
    assert np.isclose(lb.to_host(np.float32, 1)[0], np.mean(diff ** 2), rtol=1e-5)
    assert np.allclose(D.decode(gb.to_host(np.uint16, n), dt), bf(diff * 2.0 / n), rtol=1e-2, atol=0)
    # sgd: f32 master minus step, bf16 copy
    w32 = rng.standard_normal(n).astype(np.float32)
    wb, w16b = device.CudaBuffer.from_host(w32), device.CudaBuffer(n * 2)
    lib.mx_sgd_update_bf16(n, wb.ptr, dyb.ptr, w16b.ptr, ctypes.c_float(0.25), ctypes.c_float(0.5))
    device.synchronize()
    want32 = w32 - np.float32(0.125) * D.decode(dy, dt).astype(np.float32)
    got32 = wb.to_host(np.float32, n)
    assert np.array_equal(got32, want32)
    assert np.array_equal(w16b.to_host(np.uint16, n), D.encode(want32, dt))
    for x in (zb, bb, ub, ab, dyb, dub, pb, tb, gb, lb, wb, w16b):
        x.free()
    assert device.last_error() is None


def test_one_training_step_matches_f64_model(cuda):
    from maidenx_b200.mlp import Mlp
    L, Dm, B, seed, lr = 3, 256, 512, 6, 0.05
    rng = np.random.default_rng(4)
    dt = D.BF16
    x, y = H.random_store(rng, dt, B * Dm, dist="normal"), H.random_store(rng, dt, B * Dm, dist="normal")
    xb, yb = device.CudaBuffer.from_host(x), device.CudaBuffer.from_host(y)
    m = Mlp(L, Dm, B, "bf16", seed)
    # reference model in f64 from the same seeded weights (rounded to bf16 as the engine's working copy is)
    bound = 1.0 / np.sqrt(np.float32(Dm))
    W32 = [init_uniform(seed + 2 * l, Dm * Dm, bound).reshape(Dm, Dm) for l in range(L)]
    b32 = [init_uniform(seed + 2 * l + 1, 1, bound)[0] for l in range(L)]
    W = [bf(w) for w in W32]
    bs = [float(bf([b])[0]) for b in b32]
    a = [D.decode(x, dt).reshape(B, Dm)]
    us = []
    for l in range(L):
        u = bf(bf(a[-1] @ W[l].T) + bs[l])
        us.append(u)
        a.append(bf(gelu64(u)) if l < L - 1 else u)
    diff = bf(us[-1] - D.decode(y, dt).reshape(B, Dm))
    loss = np.mean(diff ** 2)
    du = bf(diff * 2.0 / (B * Dm))
    gW, gb = [None] * L, [None] * L
    for l in reversed(range(L)):
        if l < L - 1:
            du = bf(da * gelu_grad64(us[l]))
        gW[l] = du.T @ a[l]
        gb[l] = du.sum()
        da = bf(du @ W[l])
    m.train_step(xb.ptr, yb.ptr, lr)
    device.synchronize()
    assert device.last_error() is None and _lib.load().mx_tc_gemm_status() == 0
    assert np.isclose(m.loss(), loss, rtol=2e-3)
    out = D.decode(device_read(m.ptr("output"), np.uint16, B * Dm), dt).reshape(B, Dm)
    assert np.all(np.abs(out - us[-1]) <= 2e-2 * np.maximum(np.abs(us[-1]), 0.25))
    for l in range(L):
        g = D.decode(device_read(m.ptr("weight_grad", l), np.uint16, Dm * Dm), dt).reshape(Dm, Dm)
        scale = np.abs(gW[l]).max()
        assert np.all(np.abs(g - gW[l]) <= 2e-2 * np.maximum(np.abs(gW[l]), 0.1 * scale)), f"dW layer {l}"
        gbias = D.decode(device_read(m.ptr("bias_grad", l), np.uint16, 1), dt)[0]
        assert abs(gbias - gb[l]) <= 2e-2 * max(abs(gb[l]), 1e-3), f"db layer {l}"
        w_after = device_read(m.ptr("master_weight", l), np.float32, Dm * Dm).reshape(Dm, Dm)
        assert np.array_equal(w_after, W32[l] - np.float32(lr) * g.astype(np.float32)), f"SGD layer {l}"
    # the loss goes down
    first = m.loss()
    for _ in range(5):
        m.train_step(xb.ptr, yb.ptr, lr)
    assert m.loss() < first
    m.close()
    xb.free()
    yb.free()


def device_read(ptr, np_dtype, count):
    out = np.empty(count, dtype=np_dtype)
    assert _lib.load().cuda_memcpy_d2h(out.ctypes.data, ptr, out.nbytes) == 0
    return out


def test_input_pipeline_delivers_batches_in_order(cuda):
    """maidenx_b200.mlp.InputPipeline: the batch handed out by next_batch() is the one prefetched for it, also when
    the next prefetch is queued before the consumer ran (the consumer here is mx_contiguous_f32 on the op stream)."""
    import torch

    from maidenx_b200.mlp import InputPipeline
    n = 1 << 20
    like_x = torch.empty(n, dtype=torch.float32, device="cuda")
    like_y = torch.empty(n, dtype=torch.float32, device="cuda")
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    host = [(torch.full((n,), float(i)).pin_memory(), torch.full((n,), float(-i)).pin_memory()) for i in range(5)]
    pipe = InputPipeline(torch, like_x, like_y)
    fn = _lib.contiguous("f32")
    meta = np.array([n, 1, 0], dtype=np.uint64)
    seen = []
    pipe.prefetch(*host[0])
    for i in range(5):
        xb, yb = pipe.next_batch()
        if i + 1 < 5:
            pipe.prefetch(*host[i + 1])
        fn(SZ(n), SZ(1), meta.ctypes.data, xb.data_ptr(), out.data_ptr())   # consumer on the library's stream
        fn(SZ(n), SZ(1), meta.ctypes.data, yb.data_ptr(), xb.data_ptr())    # and a second one that overwrites the x buffer
        pipe.release()
        device.synchronize()
        seen.append((float(out[0]), float(out[-1]), float(xb[n // 2])))
    assert seen == [(float(i), float(i), float(-i)) for i in range(5)]
    assert device.last_error() is None


def test_one_training_step_matches_the_oracle_composed_model(cuda):
    """The engine against oracle/mlp_reference.py - the op-by-op composition on the CPU oracle that the benchmark's CPU
    arm times - from the engine's own weights: loss, network output, every gradient and the updated weights."""
    from maidenx_b200.mlp import Mlp
    from oracle import binding, mlp_reference
    L, Dm, B, seed, lr = 3, 256, 512, 9, 0.05
    rng = np.random.default_rng(8)
    dt = D.BF16
    x, y = H.random_store(rng, dt, B * Dm, dist="normal"), H.random_store(rng, dt, B * Dm, dist="normal")
    xb, yb = device.CudaBuffer.from_host(x), device.CudaBuffer.from_host(y)
    m = Mlp(L, Dm, B, "bf16", seed)
    W = [device_read(m.ptr("weight", l), np.uint16, Dm * Dm) for l in range(L)]
    b = [D.encode(device_read(m.ptr("master_bias", l), np.float32, 1), dt) for l in range(L)]
    ref = mlp_reference.CpuMlp(L, Dm, B, "bf16", [w.copy() for w in W], [v.copy() for v in b])
    binding.set_wide(True)   # f32 accumulation, as the tensor-core products and the fused passes accumulate
    try:
        loss, gWs, gbs = ref.gradients(x, y)
    finally:
        binding.set_wide(False)
    m.train_step(xb.ptr, yb.ptr, lr)
    device.synchronize()
    assert device.last_error() is None
    assert np.isclose(m.loss(), float(D.decode(loss, dt)[0]), rtol=1e-2)   # the oracle's loss is a bf16 scalar
    out = device_read(m.ptr("output"), np.uint16, B * Dm)
    H.assert_same("mlp output", dt, out, ref.last_output, float_rel=2e-2, scale=0.25, what="output")
    for l in range(L):
        g = device_read(m.ptr("weight_grad", l), np.uint16, Dm * Dm)
        # The oracle evaluates the GELU derivative as the reference's chain of ~15 elementwise ops, each rounded to bf16
        # (crates/maidenx_tensor/src/ops/unary.rs:324-346); the engine evaluates it once in f32.  The per-op 2e-2 compounds
        # along that chain, so gradients are held to 5e-2 of max(|ref|, a quarter of the largest entry).
        scale = 0.25 * np.abs(D.decode(gWs[l], dt)).max()
        H.assert_same("mlp dW", dt, g, gWs[l], float_rel=5e-2, scale=scale, what=f"dW layer {l}")
        gb = D.decode(device_read(m.ptr("bias_grad", l), np.uint16, 1), dt)[0]
        want = D.decode(gbs[l], dt)[0]
        assert abs(gb - want) <= 5e-2 * max(abs(want), 1e-3), f"db layer {l}"
    m.close()
    xb.free()
    yb.free()


@pytest.mark.parametrize("dt", [D.BF16, D.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("shape", [(256, 512, 256), (200, 264, 392), (40, 24, 56)], ids=lambda s: "x".join(map(str, s)))
def test_linear_with_bias_and_gelu_in_the_epilogue_equals_the_three_ops(cuda, dt, shape):
    """mx_linear_bias_gelu against cuda_matmul (W^T view), cuda_add (scalar bias broadcast) and cuda_gelu run one after
    the other, bit for bit - on shapes the tensor-core kernel takes (epilogue fusion) and on one it does not."""
    rows, out_f, in_f = shape
    rng = np.random.default_rng(31)
    x = H.random_store(rng, dt, rows * in_f, dist="normal")
    w = H.random_store(rng, dt, out_f * in_f, lo=-0.1, hi=0.1)
    b = H.random_store(rng, dt, 1, lo=-0.5, hi=0.5)
    meta = H.matmul_metadata([rows, out_f], [rows, in_f], [in_f, out_f], [in_f, 1], [1, in_f], 0, 0)
    z = H.run_matmul(cuda, dt, meta, rows * out_f, x, w)
    u_ref = H.run_binary(cuda, "add", dt, [rows, out_f], [out_f, 1], [0, 0], 0, 0, z, b)
    a_ref = H.run_unary(cuda, "gelu", dt, [rows * out_f], [1], 0, u_ref)
    lib = _lib.load()
    fn = getattr(lib, f"mx_linear_bias_gelu_{dt.name}")
    bufs = [device.CudaBuffer.from_host(v) for v in (x, w, b)]
    for with_act in (True, False):
        ub, ab = device.CudaBuffer.from_host(np.full(rows * out_f, 7).astype(dt.np_storage)), device.CudaBuffer.from_host(np.full(rows * out_f, 7).astype(dt.np_storage))
        fn(rows, in_f, out_f, bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, ub.ptr, ab.ptr if with_act else None)
        device.synchronize()
        assert device.last_error() is None
        H.assert_same("linear", dt, ub.to_host(dt.np_storage, rows * out_f), u_ref, what="u")
        if with_act:
            H.assert_same("linear", dt, ab.to_host(dt.np_storage, rows * out_f), a_ref, what="act")
        ub.free()
        ab.free()
    for v in bufs:
        v.free()


def test_loss_reader_returns_every_steps_loss_one_step_later(cuda):
    """maidenx_b200.mlp.LossReader against the synchronous read of a twin engine (same seed, same batch)."""
    import torch

    from maidenx_b200.mlp import LossReader, Mlp
    L, Dm, B, seed, lr = 2, 256, 256, 3, 0.05
    rng = np.random.default_rng(5)
    x, y = H.random_store(rng, D.BF16, B * Dm, dist="normal"), H.random_store(rng, D.BF16, B * Dm, dist="normal")
    xb, yb = device.CudaBuffer.from_host(x), device.CudaBuffer.from_host(y)
    a, b = Mlp(L, Dm, B, "bf16", seed), Mlp(L, Dm, B, "bf16", seed)
    want = []
    for _ in range(5):
        a.train_step(xb.ptr, yb.ptr, lr)
        want.append(a.loss())
    reader = LossReader(torch, b)
    got = []
    for i in range(5):
        b.train_step(xb.ptr, yb.ptr, lr)
        prev = reader.after_step()
        assert (prev is None) == (i == 0)
        if prev is not None:
            got.append(prev)
    got.append(reader.last())
    assert got == want and want[-1] < want[0]
    assert device.last_error() is None
    a.close()
    b.close()
    xb.free()
    yb.free()
