"""Host-side driver of the MLP training step (the data-parallel workload).

`Mlp` wraps the engine in libmaidenx_cuda.so (csrc/mlp.cu); `train_step` runs one step and,
when a torch.distributed process group is given, all-reduces each layer's gradients over NCCL
as soon as that layer's backward has been queued, so the transfer overlaps the backward of the
layers below.  Ranks hold identical weights (same seed) and different batch shards; the
gradient of the global-batch mean loss is the average of the local gradients, applied as
`grad_scale = 1 / world` inside the fused SGD update.

`DpMlp` is the NVLink-native variant: gradients and 16-bit weights live in a symmetric-memory
arena that every rank maps, and the library's own kernels (csrc/dp_sync.cu) do the exchange fused
with the optimizer step - in-switch reduction and multicast stores when the arena has a multicast
address, peer loads and stores otherwise.  torch.distributed only allocates and exchanges the
arena.  `make_mlp` picks it for world > 1 and falls back to the NCCL all-reduce driver when the
arena cannot be set up.
"""
from __future__ import annotations

import ctypes

from . import _lib

DTYPE_ID = {"bf16": 0, "f16": 1}


class Mlp:
    def __init__(self, layers: int, dim: int, batch: int, dtype: str = "bf16", seed: int = 6):
        self.lib = _lib.load()
        self.layers, self.dim, self.batch, self.dtype = layers, dim, batch, dtype
        self.h = self.lib.mx_mlp_create(layers, dim, batch, DTYPE_ID[dtype], seed)
        if not self.h:
            raise RuntimeError("mx_mlp_create failed (out of memory or bad arguments)")
        self._grad_views = None
        self.exchange = "none"

    def close(self):
        if self.h:
            self.lib.mx_mlp_destroy(self.h)
            self.h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    # --- raw phases -------------------------------------------------------------------
    def forward(self, x_ptr: int):
        self.lib.mx_mlp_forward(self.h, x_ptr)

    def loss_backward(self, y_ptr: int):
        self.lib.mx_mlp_loss_backward(self.h, y_ptr)

    def backward_layer(self, l: int):
        self.lib.mx_mlp_backward_layer(self.h, l)

    def sgd_layer(self, l: int, lr: float, grad_scale: float = 1.0):
        self.lib.mx_mlp_sgd_layer(self.h, l, lr, grad_scale)

    def loss(self) -> float:
        return float(self.lib.mx_mlp_loss(self.h))

    def ptr(self, what: str, l: int = 0) -> int:
        fn = getattr(self.lib, f"mx_mlp_{what}")
        return fn(self.h) if what in ("output", "loss_ptr") else fn(self.h, l)

    # --- torch views of the gradient buffers (for torch.distributed) ---------------------
    def grad_views(self, torch):
        """One (weight-grad, bias-grad) pair of torch tensors per layer, aliasing the engine's buffers."""
        if self._grad_views is None:
            tdt = {"bf16": torch.bfloat16, "f16": torch.float16}[self.dtype]
            views = []
            for l in range(self.layers):
                views.append((_as_tensor(torch, self.ptr("weight_grad", l), self.dim * self.dim, tdt),
                              _as_tensor(torch, self.ptr("bias_grad", l), 1, tdt)))
            self._grad_views = views
        return self._grad_views

    # --- one training step ---------------------------------------------------------------
    def train_step(self, x_ptr: int, y_ptr: int, lr: float, torch=None, dist=None, world: int = 1):
        if world <= 1:
            # one call: the optimizer update of each layer runs on a side stream beside the backward of the layers below
            self.lib.mx_mlp_train_step(self.h, x_ptr, y_ptr, lr, 1.0)
            return
        self.forward(x_ptr)
        self.loss_backward(y_ptr)
        works = []
        views = self.grad_views(torch) if world > 1 else None
        for l in reversed(range(self.layers)):
            self.backward_layer(l)
            if world > 1:
                gw, gb = views[l]
                works.append((l, dist.all_reduce(gw, async_op=True), dist.all_reduce(gb, async_op=True)))
        if world > 1:
            for l, w1, w2 in works:
                w1.wait()
                w2.wait()
                self.sgd_layer(l, lr, 1.0 / world)
        else:
            for l in range(self.layers):
                self.sgd_layer(l, lr, 1.0)

    def join(self):
        """Make the calling thread's stream wait for optimizer updates still running on the engine's side stream."""
        self.lib.mx_mlp_dp_join(self.h)


class DpMlp(Mlp):
    """Data-parallel engine over a peer-mapped arena (see csrc/dp_sync.cu).  Collective: every rank
    of the default process group must construct it, and call train_step, in the same order."""

    def __init__(self, layers: int, dim: int, batch: int, dtype: str, seed: int, torch, dist, multicast: bool = True, copy_engines: bool = False, exclusive_sms: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        self.lib = _lib.load()
        self.layers, self.dim, self.batch, self.dtype = layers, dim, batch, dtype
        self._grad_views = None
        self.h = None
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        nbytes = int(self.lib.mx_mlp_dp_arena_bytes(layers, dim))
        dev = torch.device("cuda", torch.cuda.current_device())
        self._arena = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self._hdl = symm_mem.rendezvous(self._arena, dist.group.WORLD.group_name)
        self._arena.zero_()  # barrier flags and gradient slots start from zero on every rank ...
        torch.cuda.synchronize()
        dist.barrier()       # ... before any rank's first barrier kernel can write into them
        peers = (ctypes.c_void_p * self.world)(*[int(p) for p in self._hdl.buffer_ptrs])
        mc = int(self._hdl.multicast_ptr) if multicast else 0
        self.exchange = "multimem" if mc else "peer"
        self.h = self.lib.mx_mlp_create_dp(layers, dim, batch, DTYPE_ID[dtype], seed, self.rank, self.world, peers, mc or None)
        if not self.h:
            raise RuntimeError("mx_mlp_create_dp failed (out of memory or bad arguments)")
        if copy_engines:
            if self.lib.mx_mlp_dp_set_exchange(self.h, 1, 0) != 0:
                raise RuntimeError("mx_mlp_dp_set_exchange failed (out of memory)")
            self.exchange = "copy"
        elif mc and exclusive_sms > 0:
            self.lib.mx_mlp_dp_set_exchange(self.h, 0, exclusive_sms)
            self.exchange = "multimem-exclusive"
        self.exclusive_sms = exclusive_sms if self.exchange == "multimem-exclusive" else 0
        torch.cuda.synchronize()
        dist.barrier()       # every rank's weights are initialised before anyone's first exchange

    def train_step(self, x_ptr: int, y_ptr: int, lr: float, torch=None, dist=None, world: int = 1):
        self.lib.mx_mlp_train_step_dp(self.h, x_ptr, y_ptr, lr, 1.0 / self.world)

    def join(self):
        """Make the calling thread's stream wait for the exchange of the last step (no host wait)."""
        self.lib.mx_mlp_dp_join(self.h)

    def status(self) -> int:
        """0, or 1 + the rank a barrier stopped waiting for (waits for the exchange to finish)."""
        return int(self.lib.mx_mlp_dp_status(self.h))

    def close(self):
        if self.h:
            self.lib.mx_mlp_dp_status(self.h)  # drain the side stream before the arena goes away
        super().close()
        self._hdl = None
        self._arena = None


def make_mlp(layers: int, dim: int, batch: int, dtype: str, seed: int, torch=None, dist=None, world: int = 1, exchange: str = "auto",
             exclusive_sms: int = 8):
    """The engine for `world` ranks: Mlp for one rank, DpMlp for several (exchange "auto",
    "copy", "multimem" or "peer"), Mlp driven with NCCL all-reduces for exchange == "nccl" or when the
    symmetric-memory arena cannot be set up (every rank takes the same branch: the outcome of the
    setup is agreed on with an all-reduce)."""
    if world <= 1:
        return Mlp(layers, dim, batch, dtype, seed)
    if exchange != "nccl":
        m, ok = None, 1
        if exchange == "auto":
            # two ranks: a rank's shard is half of every layer, which a few SMs cannot move in time, while the
            # exchange is short against the step - the spread peer form wins; more ranks: the multimem form on
            # SMs of its own (peer form when the arena has no multicast address)
            exchange = "peer" if world == 2 else "multimem-exclusive"
        try:
            m = DpMlp(layers, dim, batch, dtype, seed, torch, dist, multicast=exchange in ("multimem", "multimem-exclusive"),
                      copy_engines=exchange == "copy", exclusive_sms=exclusive_sms if exchange == "multimem-exclusive" else 0)
        except Exception as e:  # noqa: BLE001 - any setup failure selects the NCCL driver
            import sys
            print(f"[maidenx_b200] symmetric-memory exchange unavailable ({type(e).__name__}: {e}); using NCCL all-reduce", file=sys.stderr)
            ok = 0
        flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 1:
            return m
        if m is not None:
            m.close()
    m = Mlp(layers, dim, batch, dtype, seed)
    m.exchange = "nccl"
    return m


class InputPipeline:
    """Double-buffered host -> device input feed for a training loop.

        pipe = InputPipeline(torch, x_like, y_like)
        pipe.prefetch(host_x, host_y)
        for ...:
            xb, yb = pipe.next_batch()       # compute stream waits (on the device) for the copies of this batch
            pipe.prefetch(next_host_x, next_host_y)   # overlaps the step below
            mlp.train_step(xb.data_ptr(), yb.data_ptr(), lr, ...)
            pipe.release()                   # this batch's buffers may be refilled after the step's kernels

    Host tensors must be pinned for the copies to be asynchronous.  The compute stream is the stream the op library
    launches on (torch's current stream unless mx_set_stream chose another: pass it as `compute_stream`)."""

    def __init__(self, torch, x_like, y_like, compute_stream=None):
        self.torch = torch
        self.compute = compute_stream or torch.cuda.current_stream()
        self.copy = torch.cuda.Stream()
        self.bufs = [(x_like, y_like), (torch.empty_like(x_like), torch.empty_like(y_like))]
        self.copied = [torch.cuda.Event(), torch.cuda.Event()]
        self.consumed = [torch.cuda.Event(), torch.cuda.Event()]
        for e in self.consumed:
            e.record(self.compute)
        self.filled, self.taken = 0, 0

    def prefetch(self, host_x, host_y):
        slot = self.filled % 2
        with self.torch.cuda.stream(self.copy):
            self.copy.wait_event(self.consumed[slot])
            self.bufs[slot][0].copy_(host_x, non_blocking=True)
            self.bufs[slot][1].copy_(host_y, non_blocking=True)
            self.copied[slot].record(self.copy)
        self.filled += 1

    def next_batch(self):
        slot = self.taken % 2
        self.compute.wait_event(self.copied[slot])
        return self.bufs[slot]

    def release(self):
        self.consumed[self.taken % 2].record(self.compute)
        self.taken += 1


class LossReader:
    """Per-step loss read-back that does not stall the training loop.

        reader = LossReader(torch, mlp)
        for ...:
            mlp.train_step(...)
            prev = reader.after_step()     # loss of the PREVIOUS step (None after the first), this step's copy is queued
        final = reader.last()              # waits for the newest copy

    The 4-byte device-to-host copy of step i runs on a stream of its own behind step i (pinned destination), and the host
    collects it after it has queued step i + 1 - so the device never waits for the host between steps, which a
    synchronous read after every step forces (and which exposes whatever the step left running on side streams, such as
    the gradient exchange of its last layer).  The compute stream waits for the copy before the next step may overwrite
    the loss word."""

    def __init__(self, torch, mlp, compute_stream=None):
        self.torch = torch
        self.compute = compute_stream or torch.cuda.current_stream()
        self.stream = torch.cuda.Stream()
        self.dev = torch.as_tensor(_CudaArray(mlp.ptr("loss_ptr"), 1, "<f4"), device="cuda")
        self.host = [torch.empty(1, dtype=torch.float32).pin_memory(), torch.empty(1, dtype=torch.float32).pin_memory()]
        self.done = [torch.cuda.Event(), torch.cuda.Event()]
        self.ready = torch.cuda.Event()
        self.count = 0

    def after_step(self):
        slot = self.count % 2
        self.ready.record(self.compute)
        with self.torch.cuda.stream(self.stream):
            self.stream.wait_event(self.ready)
            self.host[slot].copy_(self.dev, non_blocking=True)
            self.done[slot].record(self.stream)
        self.compute.wait_event(self.done[slot])
        self.count += 1
        if self.count < 2:
            return None
        prev = (self.count - 2) % 2
        self.done[prev].synchronize()
        return float(self.host[prev][0])

    def last(self):
        if self.count == 0:
            return None
        slot = (self.count - 1) % 2
        self.done[slot].synchronize()
        return float(self.host[slot][0])


class _CudaArray:
    """Minimal __cuda_array_interface__ holder so torch can alias memory owned by the library."""

    def __init__(self, ptr: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


def _as_tensor(torch, ptr: int, count: int, tdt):
    # 16-bit floats travel as u16 through the array interface and are reinterpreted
    raw = torch.as_tensor(_CudaArray(ptr, count, "<i2"), device="cuda")
    return raw.view(tdt)
