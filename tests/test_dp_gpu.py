"""The NVLink data-parallel exchange (csrc/dp_sync.cu) and the data-parallel MLP engine on ONE GPU.

A single process cannot run ranks that wait for one another, so:
  * the fused "sum the ranks' gradients, update my shard, write the weights to every rank" kernel is
    run for an emulated world of 2 and 4 ranks whose arenas all live on this GPU, one rank's launch
    after the other (no launch waits for another), in its peer-pointer form, and checked bit for
    bit against numpy;
  * the flag barrier is run for world = 1 (a rank waits only for its own flag), and once with a
    peer that never arrives: the wait runs out, the kernel records the peer and returns, and the
    context stays usable;
  * the data-parallel engine with world = 1 must reproduce the single-device engine bit for bit.
The multi-GPU run of the same code (multimem and peer forms against the NCCL all-reduce driver)
is tests/dp_check.py, launched with torchrun on 2 to 8 GPUs.
"""
import ctypes

import numpy as np
import pytest

import harness as H
from maidenx_b200 import _lib, device
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu


def _read(ptr, np_dtype, count):
    out = np.empty(count, dtype=np_dtype)
    assert _lib.load().cuda_memcpy_d2h(out.ctypes.data, ptr, out.nbytes) == 0
    return out


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("dt", [D.BF16, D.F16], ids=lambda d: d.name)
def test_reduce_sgd_emulated_ranks(cuda, world, dt):
    lib = _lib.load()
    rng = np.random.default_rng(world)
    n = 8 * world * 1000          # elements of the "layer"; the shard of each rank is 8000
    shard = n // world
    grad_off, w_off, gb_off = 4096, 4096 + n * 2 + 512, 4096 + 2 * (n * 2 + 512)
    arena_bytes = gb_off + 256
    grads = [H.random_store(rng, dt, n, dist="normal") for _ in range(world)]
    gbias = [H.random_store(rng, dt, 1, dist="normal") for _ in range(world)]
    master = rng.standard_normal(n).astype(np.float32)
    mbias = np.float32(0.3)
    step = np.float32(0.05)
    arenas = []
    for p in range(world):
        host = np.zeros(arena_bytes, dtype=np.uint8)
        host[grad_off:grad_off + n * 2] = grads[p].view(np.uint8)
        host[gb_off:gb_off + 2] = gbias[p].view(np.uint8)
        arenas.append(device.CudaBuffer.from_host(host))
    peers = (ctypes.c_void_p * world)(*[a.ptr for a in arenas])
    shards, biases32, biases16 = [], [], []
    for r in range(world):
        shards.append(device.CudaBuffer.from_host(master[r * shard:(r + 1) * shard].copy()))
        biases32.append(device.CudaBuffer.from_host(np.full(64, mbias, dtype=np.float32)))
        biases16.append(device.CudaBuffer(256))
        lib.mx_dp_reduce_sgd(0 if dt is D.BF16 else 1, peers, None, None, r, world, grad_off, w_off, gb_off, shards[r].ptr, r * shard, shard,
                             biases32[r].ptr, biases16[r].ptr, ctypes.c_float(step), 0, None)
    device.synchronize()
    assert device.last_error() is None
    # expected: f32 sum in rank order, rounded to the 16-bit type, then the f32 update, then one rounding
    acc = np.zeros(n, dtype=np.float32)
    for p in range(world):
        acc = acc + D.decode(grads[p], dt).astype(np.float32)
    g16 = D.decode(D.encode(acc, dt), dt).astype(np.float32)
    want32 = master - step * g16
    want16 = D.encode(want32, dt)
    bacc = np.float32(0)
    for p in range(world):
        bacc = np.float32(bacc + np.float32(D.decode(gbias[p], dt)[0]))
    want_b32 = np.float32(mbias - step * np.float32(D.decode(D.encode([bacc], dt), dt)[0]))
    for r in range(world):
        got32 = shards[r].to_host(np.float32, shard)
        assert np.array_equal(got32, want32[r * shard:(r + 1) * shard]), f"master shard of rank {r}"
        assert biases32[r].to_host(np.float32, 1)[0] == want_b32
        assert np.array_equal(biases16[r].to_host(np.uint16, 1), D.encode([want_b32], dt).view(np.uint16))
    for p in range(world):  # every arena received every shard
        got16 = _read(arenas[p].ptr + w_off, np.uint16, n)
        assert np.array_equal(got16, want16.view(np.uint16)), f"weights in the arena of rank {p}"
    for b in arenas + shards + biases32 + biases16:
        b.free()


@pytest.mark.parametrize("world", [2, 8])
def test_reduce_sgd_staged_form_matches_peer_form(cuda, world):
    """The copy-engine route: the peers' shards are copied next to the kernel first and only the own
    arena receives the new weights.  Same sums in the same order as the peer form, so the same bits."""
    lib = _lib.load()
    dt = D.BF16
    rng = np.random.default_rng(100 + world)
    n = 8 * world * 520
    shard = n // world
    grad_off, w_off, gb_off = 4096, 4096 + n * 2 + 512, 4096 + 2 * (n * 2 + 512)
    arena_bytes = gb_off + 256
    grads = [H.random_store(rng, dt, n, dist="normal") for _ in range(world)]
    master = rng.standard_normal(n).astype(np.float32)
    step = np.float32(0.01)

    def run(staged_form):
        arenas = []
        for p in range(world):
            host = np.zeros(arena_bytes, dtype=np.uint8)
            host[grad_off:grad_off + n * 2] = grads[p].view(np.uint8)
            arenas.append(device.CudaBuffer.from_host(host))
        peers = (ctypes.c_void_p * world)(*[a.ptr for a in arenas])
        out32, out16, keep = [], [], []
        for r in range(world):
            sh = device.CudaBuffer.from_host(master[r * shard:(r + 1) * shard].copy())
            b32, b16 = device.CudaBuffer.from_host(np.zeros(64, dtype=np.float32)), device.CudaBuffer(256)
            staged = None
            if staged_form:
                bufs = [device.CudaBuffer.from_host(grads[p][r * shard:(r + 1) * shard].copy()) if p != r else None for p in range(world)]
                keep += [b for b in bufs if b is not None]
                staged = (ctypes.c_void_p * world)(*[b.ptr if b is not None else None for b in bufs])
            lib.mx_dp_reduce_sgd(0, peers, None, staged, r, world, grad_off, w_off, gb_off, sh.ptr, r * shard, shard, b32.ptr, b16.ptr,
                                 ctypes.c_float(step), 0, None)
            device.synchronize()
            out32.append(sh.to_host(np.float32, shard))
            # the staged form writes the new weights to the own arena only
            out16.append(_read(arenas[r].ptr + w_off + r * shard * 2, np.uint16, shard))
            if staged_form:
                for p in range(world):
                    if p != r:
                        assert not _read(arenas[p].ptr + w_off + r * shard * 2, np.uint16, shard).any(), "staged form wrote to a peer"
            keep += [sh, b32, b16]
        for b in arenas + keep:
            b.free()
        return out32, out16

    peer32, peer16 = run(False)
    st32, st16 = run(True)
    for r in range(world):
        assert np.array_equal(peer32[r], st32[r]) and np.array_equal(peer16[r], st16[r])
    assert device.last_error() is None


def test_barrier_world_one_and_a_peer_that_never_arrives(cuda):
    lib = _lib.load()
    arena = device.CudaBuffer.from_host(np.zeros(4096, dtype=np.uint8))
    err = device.CudaBuffer.from_host(np.zeros(64, dtype=np.uint32))
    one = (ctypes.c_void_p * 1)(arena.ptr)
    for epoch in (1, 2, 3):
        lib.mx_dp_barrier(one, 0, 0, 1, epoch, err.ptr, None)
    device.synchronize()
    assert err.to_host(np.uint32, 1)[0] == 0
    assert _read(arena.ptr, np.uint32, 1)[0] == 3
    # world = 2 with both "arenas" on this GPU and nobody playing rank 1: rank 0 posts its flag, waits
    # about two seconds for rank 1's, gives up and reports the peer; the context survives
    other = device.CudaBuffer.from_host(np.zeros(4096, dtype=np.uint8))
    two = (ctypes.c_void_p * 2)(arena.ptr, other.ptr)
    lib.mx_dp_barrier(two, 64, 0, 2, 1, err.ptr, None)
    device.synchronize()
    assert device.last_error() is None
    assert err.to_host(np.uint32, 1)[0] == 1 + 1
    assert _read(other.ptr + 64, np.uint32, 1)[0] == 1      # the flag rank 0 posted in rank 1's arena
    lib.mx_dp_barrier(one, 0, 0, 1, 4, err.ptr, None)       # still works afterwards
    device.synchronize()
    assert _read(arena.ptr, np.uint32, 1)[0] == 4
    for b in (arena, err, other):
        b.free()


def test_dp_engine_world_one_matches_single_device_engine(cuda):
    from maidenx_b200.mlp import Mlp
    lib = _lib.load()
    L, Dm, B, seed, lr = 3, 256, 512, 6, 0.05
    rng = np.random.default_rng(9)
    dt = D.BF16
    x, y = H.random_store(rng, dt, B * Dm, dist="normal"), H.random_store(rng, dt, B * Dm, dist="normal")
    xb, yb = device.CudaBuffer.from_host(x), device.CudaBuffer.from_host(y)
    ref = Mlp(L, Dm, B, "bf16", seed)
    nbytes = int(lib.mx_mlp_dp_arena_bytes(L, Dm))
    arena = device.CudaBuffer.from_host(np.zeros(nbytes, dtype=np.uint8))
    peers = (ctypes.c_void_p * 1)(arena.ptr)
    h = lib.mx_mlp_create_dp(L, Dm, B, 0, seed, 0, 1, peers, None)
    assert h
    for _ in range(3):
        ref.train_step(xb.ptr, yb.ptr, lr)
        lib.mx_mlp_train_step_dp(h, xb.ptr, yb.ptr, ctypes.c_float(lr), ctypes.c_float(1.0))
    assert lib.mx_mlp_dp_status(h) == 0
    device.synchronize()
    assert device.last_error() is None
    assert lib.mx_mlp_loss(h) == ref.loss()
    for l in range(L):
        assert np.array_equal(_read(lib.mx_mlp_weight(h, l), np.uint16, Dm * Dm), _read(ref.ptr("weight", l), np.uint16, Dm * Dm)), f"W{l}"
        assert np.array_equal(_read(lib.mx_mlp_master_weight(h, l), np.float32, Dm * Dm), _read(ref.ptr("master_weight", l), np.float32, Dm * Dm))
        assert np.array_equal(_read(lib.mx_mlp_master_bias(h, l), np.float32, 1), _read(ref.ptr("master_bias", l), np.float32, 1))
    lib.mx_mlp_destroy(h)
    ref.close()
    for b in (xb, yb, arena):
        b.free()
