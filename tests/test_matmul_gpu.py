"""Parity of matmul / matmul_backward against the CPU oracle, through the C ABI, on a B200.

Bar: integers bit-exact (wrapping); f32 / f64 bit-exact against the oracle's faithful mode
(element-type accumulation, k ascending — the SIMT kernel keeps that order and does not
contract multiplies and adds); bf16 / f16 against the oracle's wide mode (f32 accumulation,
one rounding): bit-exact on the SIMT path, within rel 2e-2 of max(|ref|, sqrt(K)) where the
tensor-core path (different summation order) takes the call.
Cases include the reference's index quirks: only strides[0] is used for the batch of
rank > 3 operands, rank-1 B is indexed by the output column alone, and terms whose linear
index reaches num_els * k are skipped (crates/maidenx_cpu/src/ops/matmul.rs:55-113).
"""
import zlib

import numpy as np
import pytest

import harness as H
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu


def zlib_seed(text):
    return zlib.crc32(text.encode())


def fwd_cases():
    """(name, out_shape, a_shape, b_shape, a_strides, b_strides, a_off, b_off, a_len, b_len)"""
    cs = H.contiguous_strides
    out = []

    def add(name, o, a, b, ast=None, bst=None, aoff=0, boff=0, alen=None, blen=None):
        ast = ast or cs(a)
        bst = bst or cs(b)
        alen = alen or (sum((d - 1) * s for d, s in zip(a, ast)) + 1 + aoff)
        blen = blen or (sum((d - 1) * s for d, s in zip(b, bst)) + 1 + boff)
        out.append((name, o, a, b, ast, bst, aoff, boff, alen, blen))

    add("mm-small", [2, 2], [2, 2], [2, 2], aoff=1, boff=1)
    add("mm-odd", [65, 33], [65, 70], [70, 33])
    add("mm-tiles", [128, 192], [128, 96], [96, 192])
    add("mm-tall-k", [7, 5], [7, 1000], [1000, 5])
    add("long-k", [3, 2], [3, 5000], [5000, 2])                            # few outputs, long reduction: one block per output element
    add("long-k-tn", [1, 3], [1, 10000], [10000, 3], ast=[1, 1])           # the weight gradient of the README example
    add("nt-linear", [50, 24], [50, 40], [40, 24], bst=[1, 40])            # x . W^T with W [24, 40]
    add("tn", [30, 20], [30, 16], [16, 20], ast=[1, 30])
    add("batched", [3, 20, 17], [3, 20, 30], [3, 30, 17])
    add("batched-span", [5, 50, 9], [5, 50, 8], [5, 8, 9])                 # 64-row tiles span batches
    add("batch-bcast-b", [4, 10, 6], [4, 10, 7], [4, 7, 6], bst=[0, 6, 1])  # B broadcast over the batch
    add("rank4", [2, 3, 4, 6], [2, 3, 4, 5], [2, 3, 5, 6])                 # batch index uses strides[0] only
    add("vec-mat", [1, 9], [1, 12], [12, 9])
    add("mat-vec", [8, 1], [8, 12], [12, 1])
    add("rank1-a", [1, 4], [5], [5, 4])                                    # contiguous formulas, m = 1
    add("rank1-b", [6, 1], [6, 5], [5])                                    # contiguous formulas, n = 1
    add("rank1-a-strided", [3, 4], [5], [5, 4], ast=[2], alen=9)           # literal: A indexed by k only, rows repeat
    add("rank1-b-strided", [6, 4], [6, 5], [4], bst=[2], blen=7)           # literal: B indexed by n only
    add("sliced-a-skips", [6, 1], [6, 4], [4, 1], ast=[16, 1])             # indices >= num_els * k are dropped
    # large enough for the tensor-core path (bf16 / f16): ragged M, N, K tiles; NT and NN operand layouts
    add("tc-nt", [200, 264], [200, 392], [392, 264], bst=[1, 392])
    add("tc-nt-tiles", [384, 512], [384, 256], [256, 512], bst=[1, 256])
    add("tc-nn", [136, 520], [136, 320], [320, 520])
    add("tc-tn", [264, 256], [264, 392], [392, 256], ast=[1, 264])          # A is the transposed view of a [392, 264] matrix
    add("tc-tt", [256, 264], [256, 384], [384, 264], ast=[1, 256], bst=[1, 384])
    # batched products on the tensor cores: dense batches, and one operand shared by every batch (stride 0), which is
    # how a [Cout, K] weight meets a [B, K, P] column buffer (crates/maidenx_tensor/src/ops/matmul.rs:161-225)
    add("tc-batched", [3, 136, 264], [3, 136, 200], [3, 200, 264])
    add("tc-batch-bcast-a", [4, 72, 264], [4, 72, 392], [4, 392, 264], ast=[0, 392, 1], alen=72 * 392)
    add("tc-batch-bcast-b-nt", [3, 200, 264], [3, 200, 392], [3, 392, 264], bst=[0, 1, 392], blen=392 * 264)
    add("tc-batched-tn", [2, 264, 256], [2, 264, 392], [2, 392, 256], ast=[392 * 264, 1, 264])
    return out


def _inputs(rng, dt, n):
    if dt.kind == "float":
        return H.random_store(rng, dt, n, dist="normal")
    return H.full_range_store(rng, dt, n)


@pytest.mark.parametrize("dt", D.ARITH, ids=lambda d: d.name)
def test_matmul_forward(oracle, cuda, dt):
    from oracle import binding
    rng = np.random.default_rng(100 + D.ARITH.index(dt))
    for name, o, a_sh, b_sh, ast, bst, aoff, boff, alen, blen in fwd_cases():
        meta = H.matmul_metadata(o, a_sh, b_sh, ast, bst, aoff, boff)
        a, b = _inputs(rng, dt, alen), _inputs(rng, dt, blen)
        n = H.numel(o)
        # f32 products large enough for the tensor cores run on split tf32 operands: summation order and the
        # last bits differ from element-type accumulation, so they are held to the stated 1e-4 against the wide oracle
        f32_tc = dt.name == "f32" and name.startswith("tc-")
        long_k = name.startswith("long-k") and dt.kind == "float"   # summed in a different order than the element-type loop
        binding.set_wide(dt.name in ("bf16", "f16") or f32_tc or long_k)
        try:
            ref = H.run_matmul(oracle, dt, meta, n, a, b)
        finally:
            binding.set_wide(False)
        got = H.run_matmul(cuda, dt, meta, n, a, b)
        if dt.name in ("bf16", "f16"):
            H.assert_same("matmul", dt, got, ref, float_rel=2e-2, what=name, scale=np.sqrt(a_sh[-1]))
        elif long_k:
            H.assert_same("matmul", dt, got, ref, float_rel=1e-4 if dt.name == "f32" else 1e-12, what=name, scale=10 * np.sqrt(a_sh[-1]))
        elif f32_tc:
            H.assert_same("matmul", dt, got, ref, float_rel=1e-4, what=name, scale=np.sqrt(a_sh[-1]))
            # split tf32 is far inside that bound (a few 1e-6: the tensor core's truncating accumulation over one
            # 128-wide K chunk); a plain tf32 product (error ~5e-4) would not pass this one
            H.assert_same("matmul", dt, got, ref, float_rel=1e-5, what=name + " (split-tf32 accuracy)", scale=np.sqrt(a_sh[-1]))
        else:
            H.assert_same("matmul", dt, got, ref, what=name)


def bwd_cases():
    """(name, out_shape, a_shape, b_shape, a_off, b_off)"""
    return [
        ("mm", [2, 2], [2, 2], [2, 2], 1, 1),
        ("mm-odd", [37, 21], [37, 45], [45, 21], 0, 0),
        ("mm-tiles", [128, 64], [128, 96], [96, 64], 0, 0),
        ("batched", [3, 10, 7], [3, 10, 12], [3, 12, 7], 2, 0),
        ("mat-vec", [9, 1], [9, 14], [14, 1], 0, 3),
        ("vec-mat", [1, 6], [1, 11], [11, 6], 0, 0),
        ("tc", [264, 256], [264, 384], [384, 256], 0, 0),   # tensor-core path for bf16 / f16
    ]


@pytest.mark.parametrize("dt", D.ARITH, ids=lambda d: d.name)
def test_matmul_backward(oracle, cuda, dt):
    from oracle import binding
    rng = np.random.default_rng(200 + D.ARITH.index(dt))
    cs = H.contiguous_strides
    for name, o, a_sh, b_sh, aoff, boff in bwd_cases():
        meta = H.matmul_metadata(o, a_sh, b_sh, cs(a_sh), cs(b_sh), aoff, boff)
        nea, neb = H.numel(a_sh), H.numel(b_sh)
        a, b, g = _inputs(rng, dt, nea + aoff), _inputs(rng, dt, neb + boff), _inputs(rng, dt, H.numel(o))
        for want_a, want_b in ((True, True), (True, False), (False, True)):
            f32_tc = dt.name == "f32" and name == "tc"
            binding.set_wide(dt.name in ("bf16", "f16") or f32_tc)
            try:
                ref = H.run_matmul_backward(oracle, dt, meta, nea, neb, g, a, b, want_a, want_b)
            finally:
                binding.set_wide(False)
            got = H.run_matmul_backward(cuda, dt, meta, nea, neb, g, a, b, want_a, want_b)
            for key in ref:
                if dt.name in ("bf16", "f16") or f32_tc:
                    k = o[-1] if key == "ga" else (o[-2] if len(o) >= 2 else 1)
                    H.assert_same("matmul_backward", dt, got[key], ref[key], float_rel=1e-4 if f32_tc else 2e-2, what=f"{name}/{key}", scale=np.sqrt(k))
                else:
                    H.assert_same("matmul_backward", dt, got[key], ref[key], what=f"{name}/{key}")


def test_matmul_backward_ignores_strides_of_a_transposed_view(oracle, cuda):
    """Linear's backward hands matmul_backward the transposed weight view; both backends read it
    as if it were contiguous (crates/maidenx_cpu/src/ops/matmul.rs:211-217)."""
    dt = D.F32
    rng = np.random.default_rng(5)
    o, a_sh, b_sh = [6, 4], [6, 5], [5, 4]
    meta = H.matmul_metadata(o, a_sh, b_sh, [5, 1], [1, 5], 0, 0)  # B = W^T view, strides [1, 5]
    a, b, g = _inputs(rng, dt, 30), _inputs(rng, dt, 20), _inputs(rng, dt, 24)
    ref = H.run_matmul_backward(oracle, dt, meta, 30, 20, g, a, b)
    got = H.run_matmul_backward(cuda, dt, meta, 30, 20, g, a, b)
    for key in ref:
        H.assert_same("matmul_backward", dt, got[key], ref[key], what=key)


def test_matmul_backward_scalar_grad(oracle, cuda):
    """out_ndim == 0: every gradient row is grad_output[0] times the other operand (matmul.rs:204-207,240-243)."""
    dt = D.F32
    rng = np.random.default_rng(6)
    meta = [0, 1, 1, 7, 7, 1, 1, 0, 0]  # out_ndim 0, a_shape [7], b_shape [7]
    a, b, g = _inputs(rng, dt, 7), _inputs(rng, dt, 7), _inputs(rng, dt, 1)
    ref = H.run_matmul_backward(oracle, dt, meta, 7, 7, g, a, b)
    got = H.run_matmul_backward(cuda, dt, meta, 7, 7, g, a, b)
    for key in ref:
        H.assert_same("matmul_backward", dt, got[key], ref[key], what=key)


# ---------------------------------------------------------------------------------------
# Tensor-core kernel at benchmark scale: more output tiles than SMs (every CTA walks its
# persistent loop several times, both TMEM accumulators change hands), K = 8192 (128
# k-blocks through the 4-stage ring), a ragged last row-group and ragged edge tiles.
# The oracle's matmul is row-independent, so it is run on a sample of rows only.
# ---------------------------------------------------------------------------------------
def _sample_rows(m, count=32):
    edge = [0, 1, 127, 128, 129, m // 2, m - 129, m - 128, m - 2, m - 1]
    rows = sorted({r for r in edge if 0 <= r < m})
    rng = np.random.default_rng(m)
    while len(rows) < count:
        r = int(rng.integers(0, m))
        if r not in rows:
            rows.append(r)
    return np.array(sorted(rows))


BIG_FWD = [
    # name, M, N, K, a_major, b_major  ("k": K contiguous, "mn": M / N contiguous)
    ("nt-512-tiles", 4096, 4096, 8192, "k", "k"),
    ("nn-512-tiles", 4096, 4096, 8192, "k", "mn"),
    ("tn-512-tiles", 4096, 4096, 8192, "mn", "mn"),
    ("nt-ragged-group", 2216, 840, 8192, "k", "k"),      # 18 row-tiles: the last group of 16 holds two; 40-row and 72-column edge tiles
    ("tt-ragged", 2216, 840, 4104, "mn", "k"),           # ragged K block (4104 = 64 * 64 + 8)
    # few tiles, long reduction: K is cut into slices that run as batches, f32 partials summed by a second kernel
    ("splitk-nt", 200, 264, 32768, "k", "k"),
    ("splitk-tn", 264, 256, 65536, "mn", "mn"),          # the shape class of the conv weight gradient
]


@pytest.mark.parametrize("dt", [D.BF16, D.F16, D.F32], ids=lambda d: d.name)
@pytest.mark.parametrize("case", BIG_FWD, ids=lambda c: c[0])
def test_matmul_forward_many_tiles(oracle, cuda, dt, case):
    from oracle import binding
    name, m, n, k, amaj, bmaj = case
    rng = np.random.default_rng(zlib_seed(name + dt.name))
    a = H.random_store(rng, dt, m * k, dist="normal")
    b = H.random_store(rng, dt, k * n, dist="normal")
    ast = [k, 1] if amaj == "k" else [1, m]
    bst = [1, k] if bmaj == "k" else [n, 1]
    meta = H.matmul_metadata([m, n], [m, k], [k, n], ast, bst, 0, 0)
    got = H.run_matmul(cuda, dt, meta, m * n, a, b).reshape(m, n)
    rows = _sample_rows(m)
    a_rows = (a.reshape(m, k)[rows] if amaj == "k" else a.reshape(k, m)[:, rows].T).copy().reshape(-1)
    smeta = H.matmul_metadata([len(rows), n], [len(rows), k], [k, n], [k, 1], bst, 0, 0)
    binding.set_wide(True)
    try:
        ref = H.run_matmul(oracle, dt, smeta, len(rows) * n, a_rows, b).reshape(len(rows), n)
    finally:
        binding.set_wide(False)
    rel = 2e-2 if dt.name in ("bf16", "f16") else 1e-4
    H.assert_same("matmul", dt, got[rows].reshape(-1), ref.reshape(-1), float_rel=rel, what=name, scale=np.sqrt(k))


@pytest.mark.parametrize("dt", [D.BF16, D.F16, D.F32], ids=lambda d: d.name)
def test_matmul_backward_many_tiles(oracle, cuda, dt):
    """grad_a = g . B^T (reduction over n) and grad_b = A^T . g (reduction over m) with more tiles than SMs."""
    from oracle import binding
    m, k, n = 2216, 4096, 840
    rng = np.random.default_rng(zlib_seed("bwd" + dt.name))
    a = H.random_store(rng, dt, m * k, dist="normal")
    b = H.random_store(rng, dt, k * n, dist="normal")
    g = H.random_store(rng, dt, m * n, dist="normal")
    meta = H.matmul_metadata([m, n], [m, k], [k, n], [k, 1], [n, 1], 0, 0)
    got = H.run_matmul_backward(cuda, dt, meta, m * k, k * n, g, a, b)
    ga, gb = got["ga"].reshape(m, k), got["gb"].reshape(k, n)
    rel = 2e-2 if dt.name in ("bf16", "f16") else 1e-4
    binding.set_wide(True)
    try:
        rows = _sample_rows(m)
        smeta = H.matmul_metadata([len(rows), n], [len(rows), k], [k, n], [k, 1], [n, 1], 0, 0)
        ref = H.run_matmul_backward(oracle, dt, smeta, len(rows) * k, k * n, g.reshape(m, n)[rows].copy().reshape(-1),
                                    np.zeros(len(rows) * k, dt.np_storage), b, want_b=False)["ga"]
        H.assert_same("matmul_backward", dt, ga[rows].reshape(-1), ref, float_rel=rel, what="ga", scale=np.sqrt(n))
        cols = _sample_rows(k)
        smeta = H.matmul_metadata([m, n], [m, len(cols)], [len(cols), n], [len(cols), 1], [n, 1], 0, 0)
        ref = H.run_matmul_backward(oracle, dt, smeta, m * len(cols), len(cols) * n, g, a.reshape(m, k)[:, cols].copy().reshape(-1),
                                    np.zeros(len(cols) * n, dt.np_storage), want_a=False)["gb"]
        H.assert_same("matmul_backward", dt, gb[cols].reshape(-1), ref, float_rel=rel, what="gb", scale=np.sqrt(m))
    finally:
        binding.set_wide(False)


def test_stale_device_wait_report_is_surfaced_and_does_not_poison_later_products(oracle, cuda):
    """A tensor-core kernel whose bounded wait ran out leaves a word in device memory.  The ABI's own
    synchronisation points must report it (callers of the reference ABI never call the mx_* status functions),
    and launches made while the word is still there must compute their product normally.  The word is written
    from the host: no wait has to run out on the GPU."""
    import ctypes
    from maidenx_b200 import _lib, device
    from oracle import binding
    lib = _lib.load()
    poke = lib.mx_debug_tc_gemm_poke_status
    poke.argtypes, poke.restype = [ctypes.c_int], ctypes.c_int
    dt = D.BF16
    rng = np.random.default_rng(77)
    m, n, k = 256, 512, 256
    a, b = H.random_store(rng, dt, m * k, dist="normal"), H.random_store(rng, dt, k * n, dist="normal")
    meta = H.matmul_metadata([m, n], [m, k], [k, n], [k, 1], [1, k], 0, 0)
    binding.set_wide(True)
    try:
        ref = H.run_matmul(oracle, dt, meta, m * n, a, b)
    finally:
        binding.set_wide(False)
    assert poke(3) == 0
    bufs = [device.CudaBuffer.from_host(x) for x in (a, b, np.zeros(m * n, dt.np_storage))]
    try:
        device.dispatch("matmul", dt.name, meta, ctypes.c_size_t(m * n), "META", bufs[0].ptr, bufs[1].ptr, bufs[2].ptr)
        out = np.empty(m * n, dt.np_storage)
        rc = lib.cuda_memcpy_d2h(out.ctypes.data, bufs[2].ptr, out.nbytes)
        assert rc != 0, "the copy that follows the product must report the device-side wait"
        assert lib.mx_last_error() == 5 and lib.mx_last_cuda_error() == 3
        lib.mx_clear_error()
        H.assert_same("matmul", dt, out, ref, float_rel=2e-2, what="product launched over a stale report", scale=np.sqrt(k))
        assert lib.cuda_memcpy_d2h(out.ctypes.data, bufs[2].ptr, out.nbytes) == 0  # reported once, then clear
        assert lib.mx_tc_gemm_status() == 0
    finally:
        lib.mx_clear_error()
        for x in bufs:
            x.free()


@pytest.mark.parametrize("dt", [D.BF16, D.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("case", BIG_FWD, ids=lambda c: c[0])
def test_two_cta_kernel_matches_too(oracle, cuda, dt, case):
    """mx_set_gemm_cta_group(2): pairs of CTAs share the B tile (tcgen05.mma.cta_group::2, matmul_tc2.cu).  Same products
    as the default one-CTA kernel, on every many-tile case: odd numbers of row tiles (a pair with an empty half),
    ragged edges, both operand majors, split-K."""
    from maidenx_b200 import _lib
    lib = _lib.load()
    lib.mx_set_gemm_cta_group(2)
    try:
        test_matmul_forward_many_tiles(oracle, cuda, dt, case)
    finally:
        lib.mx_set_gemm_cta_group(1)


@pytest.mark.parametrize("dt", [D.BF16, D.F16], ids=lambda d: d.name)
def test_two_cta_kernel_on_the_small_batched_and_backward_cases(oracle, cuda, dt):
    from maidenx_b200 import _lib
    lib = _lib.load()
    lib.mx_set_gemm_cta_group(2)
    try:
        test_matmul_forward(oracle, cuda, dt)
        test_matmul_backward(oracle, cuda, dt)
    finally:
        lib.mx_set_gemm_cta_group(1)


SHORT_K = [
    ("keepb-nt", 25640, 600, 256, "k", "k"),      # 201 row tiles (40-row edge), 3 column tiles (88-column edge): 49 CTAs per column tile
    ("keepb-nn", 25640, 600, 256, "k", "mn"),
    ("keepb-tn", 25640, 600, 192, "mn", "mn"),    # three k-blocks: the ring is three slots long
    ("keepb-ragged-k", 25640, 520, 136, "k", "k"),
    ("keepb-one-kb", 151 * 128, 2304, 64, "k", "mn"),
]


@pytest.mark.parametrize("dt", [D.BF16, D.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("case", SHORT_K, ids=lambda c: c[0])
def test_short_reductions_with_the_b_panel_resident(oracle, cuda, dt, case):
    """K <= 256 with many row tiles: the CTAs of a column tile load its B panel once and stream only A.  Against the
    oracle on sampled rows, and bit for bit against the general schedule of the same kernel."""
    from maidenx_b200 import _lib
    lib = _lib.load()
    name, m, n, k, amaj, bmaj = case
    assert lib.mx_debug_gemm_keep_b_ctas((m + 127) // 128, (n + 255) // 256, (k + 63) // 64, 1, 148) > 0
    test_matmul_forward_many_tiles(oracle, cuda, dt, case)
    rng = np.random.default_rng(zlib_seed(name))
    a = H.random_store(rng, dt, m * k, dist="normal")
    b = H.random_store(rng, dt, k * n, dist="normal")
    meta = H.matmul_metadata([m, n], [m, k], [k, n], [k, 1] if amaj == "k" else [1, m], [1, k] if bmaj == "k" else [n, 1], 0, 0)
    kept = H.run_matmul(cuda, dt, meta, m * n, a, b)
    lib.mx_debug_set_gemm_keep_b(0)
    try:
        general = H.run_matmul(cuda, dt, meta, m * n, a, b)
    finally:
        lib.mx_debug_set_gemm_keep_b(1)
    assert np.array_equal(kept, general)
