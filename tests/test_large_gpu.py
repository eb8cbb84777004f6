"""More than 2^32 elements in one call (64-bit indexing): the saturating u8 add over a flat tensor of 2^32 + 4099
elements and the wrapping u8 sum of all of it, checked on the device against torch arithmetic (the CPU oracle
would need minutes and three 4 GiB host copies).  About 50 GB of the 180 GB of HBM at the peak (the index
tensor the inputs are derived from is 34 GB)."""
import ctypes

import numpy as np
import pytest

from maidenx_b200 import _lib, device

pytestmark = pytest.mark.gpu
SZ = ctypes.c_size_t


def test_flat_add_and_full_sum_beyond_32_bit_counts(cuda):
    import torch
    n = (1 << 32) + 4099
    idx = torch.arange(n, device="cuda", dtype=torch.int64)
    a = (idx % 251).to(torch.uint8)
    b = ((idx * 7) % 13).to(torch.uint8)
    del idx
    out = torch.empty(n, device="cuda", dtype=torch.uint8)
    meta = np.array([n, 1, 1, 0, 0], dtype=np.uint64)
    _lib.op("add", "u8")(SZ(n), SZ(1), meta.ctypes.data, a.data_ptr(), b.data_ptr(), out.data_ptr())
    device.synchronize()
    assert device.last_error() is None
    # chunked comparison keeps the temporaries small
    step = 1 << 28
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        want = torch.clamp(a[lo:hi].to(torch.int16) + b[lo:hi].to(torch.int16), max=255).to(torch.uint8)  # u8 add saturates
        assert torch.equal(out[lo:hi], want), f"mismatch in [{lo}, {hi})"
    # sum of everything, wrapping in u8 (the reference's integer sums wrap)
    total = int(a.sum(dtype=torch.int64).item())
    res = torch.full((8,), 7, device="cuda", dtype=torch.uint8)
    rmeta = np.array([n, 1, n, 1, 0], dtype=np.uint64)
    _lib.op("sum", "u8")(SZ(n), SZ(1), SZ(1), rmeta.ctypes.data, a.data_ptr(), res.data_ptr())
    device.synchronize()
    assert device.last_error() is None
    assert int(res[0].item()) == total % 256 and int(res[1].item()) == 7
