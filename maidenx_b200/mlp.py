"""Host-side driver of the MLP training step (the data-parallel workload).

`Mlp` wraps the engine in libmaidenx_cuda.so (csrc/mlp.cu); `train_step` runs one step and,
when a torch.distributed process group is given, all-reduces each layer's gradients over NCCL
as soon as that layer's backward has been queued, so the transfer overlaps the backward of the
layers below.  Ranks hold identical weights (same seed) and different batch shards; the
gradient of the global-batch mean loss is the average of the local gradients, applied as
`grad_scale = 1 / world` inside the fused SGD update.
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


class _CudaArray:
    """Minimal __cuda_array_interface__ holder so torch can alias memory owned by the library."""

    def __init__(self, ptr: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


def _as_tensor(torch, ptr: int, count: int, tdt):
    # 16-bit floats travel as u16 through the array interface and are reinterpreted
    raw = torch.as_tensor(_CudaArray(ptr, count, "<i2"), device="cuda")
    return raw.view(tdt)
