"""Parity of the strided elementwise families (binary, in-place, unary, unary-with-constant)
against the CPU oracle, through the C ABI, on a B200.

Bar: bit-exact for bool / integer outputs and for float ops whose arithmetic is IEEE-exact
(+ - * / sqrt min max compare ...); transcendental float ops within f32 rel 1e-5
(f64 1e-12, bf16/f16 1e-2 = about one unit in the last place of the 16-bit result).
Layouts cover every kernel of the engine: flat (with tail), row broadcasts, transposed
tiles with and without vector alignment, permuted 3-D (generic), offset-1 views like the
reference's fixtures, scalars (num_dims = 0) and NULL metadata.
"""
import zlib

import numpy as np
import pytest

import harness as H
from maidenx_b200 import _signatures as sig
from maidenx_b200 import dtypes as D

pytestmark = pytest.mark.gpu

TRANSCENDENTAL = {"sigmoid", "tanh", "gelu", "sin", "cos", "tan", "ln", "log10", "log2", "exp", "exp10", "exp2",
                  "softplus", "pow", "elu"}
POSITIVE_DOMAIN = {"ln", "log10", "log2"}


def float_tol(op, dt):
    if op not in TRANSCENDENTAL or dt.kind != "float":
        return 0.0
    return {"f32": 1e-5, "f64": 1e-12, "bf16": 1e-2, "f16": 1e-2}[dt.name]


def layouts(rng):
    """(name, dims, lhs_strides, rhs_strides, lhs_off, rhs_off, lhs_len, rhs_len)"""
    out = []
    n = 10007
    out.append(("flat", [n], [1], [1], 0, 0, n, n))
    out.append(("flat-aligned-offset", [4096], [1], [1], 16, 32, 4096 + 16, 4096 + 32))
    out.append(("offset1", [n], [1], [1], 1, 1, n + 2, n + 2))
    r, c = 37, 264
    out.append(("2d-merged", [r, c], [c, 1], [c, 1], 0, 0, r * c, r * c))
    out.append(("row-bcast-rhs", [r, c], [c, 1], [0, 1], 0, 0, r * c, c))
    out.append(("col-bcast-rhs", [r, c], [c, 1], [1, 0], 0, 0, r * c, r))
    out.append(("scalar-bcast-rhs", [r, c], [c, 1], [0, 0], 0, 3, r * c, 8))
    out.append(("padded-rows", [r, c], [c + 16, 1], [c, 1], 0, 0, r * (c + 16), r * c))
    out.append(("transposed-lhs-vec", [128, 192], [1, 128], [192, 1], 0, 0, 128 * 192, 128 * 192))
    out.append(("transposed-lhs-odd", [67, 131], [1, 67], [131, 1], 0, 0, 67 * 131, 67 * 131))
    out.append(("transposed-both", [96, 80], [1, 96], [1, 96], 0, 0, 96 * 80, 96 * 80))
    out.append(("transposed-lhs-bcast-rhs", [70, 90], [1, 70], [0, 1], 1, 0, 70 * 90 + 1, 90))
    out.append(("batched-transpose", [3, 40, 72], [40 * 72, 1, 40], [40 * 72, 72, 1], 0, 0, 3 * 40 * 72, 3 * 40 * 72))
    out.append(("permuted-3d", [5, 6, 7], [1, 35, 5], [42, 7, 1], 0, 0, 210, 210))
    out.append(("size1-dims", [1, 9, 1, 11], [99, 11, 11, 1], [0, 11, 0, 1], 0, 0, 99, 99))
    out.append(("scalar", [], [], [], 2, 1, 4, 4))
    return out


@pytest.mark.parametrize("op", sig.BINARY_ARITH + sig.BINARY_BOOL)
def test_binary(oracle, cuda, op):
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    dts = D.ALL if op in sig.BINARY_BOOL else D.ARITH
    for dt in dts:
        for name, dims, ls, rs, lo, ro, ll, rl in layouts(rng):
            lhs, rhs = H.full_range_store(rng, dt, ll), H.full_range_store(rng, dt, rl)
            if dt.kind != "float":  # make equal / zero pairs common enough to matter
                k = min(ll, rl) // 3
                rhs[:k] = lhs[:k]
            ref = H.run_binary(oracle, op, dt, dims, ls, rs, lo, ro, lhs, rhs)
            got = H.run_binary(cuda, op, dt, dims, ls, rs, lo, ro, lhs, rhs)
            H.assert_same(op, dt, got, ref, what=name)
        # NULL metadata = contiguous, no offsets (crates/maidenx_cuda/kernels/ops/binary.cu:20-25)
        lhs, rhs = H.full_range_store(rng, dt, 5000), H.full_range_store(rng, dt, 5000)
        ref = H.run_binary(oracle, op, dt, [5000], [1], [1], 0, 0, lhs, rhs, null_meta=True)
        got = H.run_binary(cuda, op, dt, [5000], [1], [1], 0, 0, lhs, rhs, null_meta=True)
        H.assert_same(op, dt, got, ref, what="null-meta")


def inplace_layouts():
    """(name, dims, lhs_strides, rhs_strides, lhs_off, rhs_off, lhs_len, rhs_len)"""
    return [
        ("flat", [9001], [1], [1], 0, 0, 9001, 9001),
        ("offset1", [513], [1], [1], 1, 1, 515, 515),
        ("lhs-transposed", [64, 96], [1, 64], [96, 1], 0, 0, 64 * 96, 64 * 96),
        ("lhs-transposed-odd", [33, 77], [1, 33], [77, 1], 2, 0, 33 * 77 + 2, 33 * 77),
        ("rhs-bcast", [20, 48], [48, 1], [0, 1], 0, 0, 960, 48),
        ("lhs-strided-rows", [10, 16], [32, 1], [16, 1], 0, 0, 320, 160),
        ("lhs-permuted-3d", [4, 5, 6], [1, 24, 4], [30, 6, 1], 0, 0, 120, 120),
        # an lhs that overlaps itself: every logical row lands on the same 8 elements, applied in order
        ("lhs-stride0", [5, 8], [0, 1], [8, 1], 0, 0, 8, 40),
        ("scalar", [], [], [], 1, 0, 3, 3),
    ]


@pytest.mark.parametrize("op", sig.BINARY_INPLACE)
def test_binary_inplace(oracle, cuda, op):
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    for dt in D.ARITH:
        for name, dims, ls, rs, lo, ro, ll, rl in inplace_layouts():
            if name == "lhs-stride0" and dt.kind == "float":
                lhs, rhs = H.random_store(rng, dt, ll), H.random_store(rng, dt, rl, lo=0.5, hi=1.5)
            else:
                lhs, rhs = H.full_range_store(rng, dt, ll), H.full_range_store(rng, dt, rl)
            ref = H.run_binary_inplace(oracle, op, dt, dims, ls, rs, lo, ro, lhs, rhs)
            got = H.run_binary_inplace(cuda, op, dt, dims, ls, rs, lo, ro, lhs, rhs)
            H.assert_same(op, dt, got, ref, what=name)  # whole buffer: untouched elements must stay untouched


def unary_layouts():
    """(name, dims, strides, off, buffer_len)"""
    return [
        ("flat", [10007], [1], 0, 10007),
        ("offset1", [1000], [1], 1, 1002),
        ("transposed-vec", [128, 64], [1, 128], 0, 8192),
        ("transposed-odd", [45, 83], [1, 45], 3, 45 * 83 + 3),
        ("bcast-row", [33, 64], [0, 1], 0, 64),       # a lone broadcast input: strides [0, 1]
        ("bcast-col", [33, 64], [1, 0], 0, 33),
        ("padded-rows", [12, 40], [48, 1], 0, 576),
        ("permuted-3d", [5, 6, 7], [1, 35, 5], 0, 210),
        ("every-other", [777], [2], 0, 1554),
        ("scalar", [], [], 2, 4),
    ]


def unary_input(rng, op, dt, count):
    if dt.kind == "float":
        if op in POSITIVE_DOMAIN:
            return H.random_store(rng, dt, count, lo=0.01, hi=10.0)
        if op in TRANSCENDENTAL:
            return H.random_store(rng, dt, count, lo=-4.0, hi=4.0)
    return H.full_range_store(rng, dt, count)


UNARY_TABLE = [(op, fam, d) for op, d, fam in sig.op_table() if fam in ("unary", "unary_bool")]


@pytest.mark.parametrize("op", sorted({op for op, _, _ in UNARY_TABLE}))
def test_unary(oracle, cuda, op):
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    for dt in [d for o, _, d in UNARY_TABLE if o == op]:
        for name, dims, st, off, blen in unary_layouts():
            x = unary_input(rng, op, dt, blen)
            ref = H.run_unary(oracle, op, dt, dims, st, off, x)
            got = H.run_unary(cuda, op, dt, dims, st, off, x)
            scale = None
            if op == "gelu":  # cancels against |x|
                scale = D.decode(H.run_unary(oracle, "abs", dt, dims, st, off, x), dt)
            elif op == "softplus":  # ln(1 + exp(x)) rounds 1 + exp(x) first
                scale = 1.0
            H.assert_same(op, dt, got, ref, float_rel=float_tol(op, dt), what=name, scale=scale)
        x = unary_input(rng, op, dt, 3000)
        ref = H.run_unary(oracle, op, dt, [3000], [1], 0, x, null_meta=True)
        got = H.run_unary(cuda, op, dt, [3000], [1], 0, x, null_meta=True)
        H.assert_same(op, dt, got, ref, float_rel=float_tol(op, dt), what="null-meta",
                      scale=D.decode(x, dt) if op == "gelu" else (1.0 if op == "softplus" else None))


CONST_TABLE = [(op, fam, d) for op, d, fam in sig.op_table() if fam in ("unary_const", "unary_const_bool")]


def constants_for(op, dt):
    if dt.kind == "bool":
        return [True, False]
    if dt.kind == "float":
        if op == "pow":
            return [2.0, 0.5, -1.0, 3.0]
        return [0.0, 1.5, -2.25, 0.1]
    info = np.iinfo(dt.np_storage)
    cs = [0, 1, 3, info.max, info.max // 3]
    if dt.kind == "sint":
        cs += [-1, -2, info.min]
    if op == "pow":
        cs = [0, 1, 2, 3, 5, 7, 13, 40, 63, 64, 65] + ([-1, -2, -3] if dt.kind == "sint" else [])
        cs = [c for c in cs if info.min <= c <= info.max]
    return cs


@pytest.mark.parametrize("op", sorted({op for op, _, _ in CONST_TABLE}))
def test_unary_with_constant(oracle, cuda, op):
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    for dt in [d for o, _, d in CONST_TABLE if o == op]:
        for c in constants_for(op, dt):
            for name, dims, st, off, blen in unary_layouts()[:6] + unary_layouts()[-1:]:
                if dt.kind == "float" and op == "pow":
                    x = H.random_store(rng, dt, blen, lo=0.1, hi=4.0)
                elif dt.kind == "float" and op == "elu":
                    x = H.random_store(rng, dt, blen, lo=-4.0, hi=4.0)
                else:
                    x = H.full_range_store(rng, dt, blen)
                    if dt.kind in ("uint", "sint") and op == "pow":  # small bases too, so powers stay in range
                        small = rng.integers(-3 if dt.kind == "sint" else 0, 12, blen // 2)
                        x[: blen // 2] = small.astype(dt.np_storage)
                ref = H.run_unary(oracle, op, dt, dims, st, off, x, scalar=c)
                got = H.run_unary(cuda, op, dt, dims, st, off, x, scalar=c)
                H.assert_same(op, dt, got, ref, float_rel=float_tol(op, dt), what=f"{name} c={c}",
                              scale=abs(c) if op == "elu" else None)  # alpha * (exp(x) - 1) cancels against alpha


def test_host_metadata_matches_device_metadata(oracle, cuda, cuda_hostmeta):
    """The metadata pointer may be device memory (the reference's convention) or host memory."""
    rng = np.random.default_rng(7)
    dt = D.F32
    lhs, rhs = H.random_store(rng, dt, 67 * 131), H.random_store(rng, dt, 67 * 131)
    a = H.run_binary(cuda, "add", dt, [67, 131], [1, 67], [131, 1], 0, 0, lhs, rhs)
    b = H.run_binary(cuda_hostmeta, "add", dt, [67, 131], [1, 67], [131, 1], 0, 0, lhs, rhs)
    c = H.run_binary(oracle, "add", dt, [67, 131], [1, 67], [131, 1], 0, 0, lhs, rhs)
    assert np.array_equal(a, b) and np.array_equal(a, c)


def test_metadata_uploaded_outside_the_wrappers(cuda):
    """A metadata block the side table has never seen is read back from the device."""
    import ctypes
    from maidenx_b200 import _lib, device
    lib = _lib.load()
    n = 1000
    rng = np.random.default_rng(3)
    x = rng.standard_normal(n + 1).astype(np.float32)
    meta = np.array([n, 1, 1], dtype=np.uint64)  # dims | strides | offset = 1
    mbuf = device.CudaBuffer(meta.nbytes)
    # stage through a second device buffer so cuda_memcpy_h2d never sees the final address
    stage = device.CudaBuffer.from_host(np.concatenate([meta, meta]))  # 48 bytes: a different block
    assert lib.cuda_memcpy_d2d(mbuf.ptr, stage.ptr, meta.nbytes) == 0
    xin, out = device.CudaBuffer.from_host(x), device.CudaBuffer(n * 4)
    _lib.op("neg", "f32")(ctypes.c_size_t(n), ctypes.c_size_t(1), mbuf.ptr, xin.ptr, out.ptr)
    assert device.last_error() is None
    assert np.array_equal(out.to_host(np.float32, n), -x[1:])
    for b in (mbuf, stage, xin, out):
        b.free()


def test_inconsistent_metadata_is_reported(cuda):
    from maidenx_b200 import device
    rng = np.random.default_rng(1)
    x = H.random_store(rng, D.F32, 100)
    with pytest.raises(device.CudaError):
        # dims say 10 x 9 = 90 elements, num_els says 100
        be = cuda
        n = 100

        def build(put, META):
            import ctypes
            a, _ = put(x)
            b, _ = put(x)
            o, oh = put(np.zeros(n, np.float32))
            return [ctypes.c_size_t(n), ctypes.c_size_t(2), META, a, b, o], {"out": (oh, np.float32, n)}

        be.call("add", D.F32, [10, 9, 9, 1, 9, 1, 0, 0], build)


@pytest.mark.parametrize("op", ["add", "sub", "div", "mul"])
def test_16bit_float_arithmetic_is_bit_exact_on_random_bit_patterns(oracle, cuda, op):
    """bf16 / f16 add and sub run on the packed 16-bit adder and div on the approximate reciprocal
    with an exact fallback near rounding midpoints; both must give the bits of "compute in f32,
    round once" that the CPU backend produces.  Operands are raw random bit patterns (every
    exponent, subnormals, infinities, NaNs) plus pairs constructed to have close exponents,
    where sums cancel and quotients land near 1."""
    rng = np.random.default_rng(17 + len(op))
    n = 1 << 21
    for dt in (D.BF16, D.F16):
        a = rng.integers(0, 1 << 16, n, dtype=np.uint16)
        b = rng.integers(0, 1 << 16, n, dtype=np.uint16)
        # second half: b = a with the low mantissa bits and the sign re-drawn -> same or adjacent binade
        h = n // 2
        low_bits = 8 if dt is D.BF16 else 11
        b[h:] = (a[h:] & np.uint16(0x7FFF & ~((1 << low_bits) - 1))) | rng.integers(0, 1 << low_bits, n - h, dtype=np.uint16) \
            | (rng.integers(0, 2, n - h, dtype=np.uint16) << np.uint16(15))
        a, b = a.view(dt.np_storage), b.view(dt.np_storage)
        ref = H.run_binary(oracle, op, dt, [n], [1], [1], 0, 0, a, b)
        got = H.run_binary(cuda, op, dt, [n], [1], [1], 0, 0, a, b)
        H.assert_same(op, dt, got, ref, what="bit-patterns")
        # the strided kernels share the packed cores: a transposed view of the same data
        r, c = 1024, n // 1024
        ref = H.run_binary(oracle, op, dt, [r, c], [1, r], [c, 1], 0, 0, a, b)
        got = H.run_binary(cuda, op, dt, [r, c], [1, r], [c, 1], 0, 0, a, b)
        H.assert_same(op, dt, got, ref, what="bit-patterns-transposed")


def test_small_block_pool_reuses_slots_and_can_be_switched_off(cuda):
    """cuda_malloc of a metadata-sized block comes from the pool: freeing and allocating again returns the same
    slot, slots of one slab are 2 KB apart, and a large request bypasses the pool."""
    import ctypes

    from maidenx_b200 import _lib
    lib = _lib.load()

    def alloc(n):
        p = ctypes.c_void_p()
        assert lib.cuda_malloc(ctypes.byref(p), n) == 0
        return p.value

    lib.mx_set_small_pool(1)
    a, b = alloc(40), alloc(2048)
    assert abs(a - b) % 2048 == 0
    assert lib.cuda_free(a) == 0
    c = alloc(16)
    assert c == a                      # the freed slot is handed out again
    big = alloc(1 << 20)
    assert lib.cuda_free(big) == 0 and lib.cuda_free(b) == 0 and lib.cuda_free(c) == 0
    # ops keep working on pooled metadata blocks (the whole suite runs that way); with the pool off as well
    lib.mx_set_small_pool(0)
    try:
        d = alloc(40)
        assert lib.cuda_free(d) == 0
        rng = np.random.default_rng(0)
        x, y = H.random_store(rng, D.F32, 100), H.random_store(rng, D.F32, 100)
        got = H.run_binary(cuda, "add", D.F32, [100], [1], [1], 0, 0, x, y)
        assert np.array_equal(got, x + y)
    finally:
        lib.mx_set_small_pool(1)


def test_caching_allocator_size_classes_and_side_table_ranges(cuda):
    """Blocks above the 2 KB slots are cached by power-of-two size class; requests above 64 MB bypass the cache.
    A metadata-sized upload into the interior of an allocation is forgotten when the allocation is freed or when a
    copy through the wrappers overwrites it (a stale entry would hand an op the old dims and strides)."""
    import ctypes

    from maidenx_b200 import _lib
    lib = _lib.load()

    def alloc(n):
        p = ctypes.c_void_p()
        assert lib.cuda_malloc(ctypes.byref(p), n) == 0
        return p.value

    lib.mx_set_small_pool(1)
    a = alloc(100000)                      # class 2^17
    assert lib.cuda_free(a) == 0
    b = alloc(70000)                       # same class: the cached block comes back
    assert b == a
    c = alloc(100000)
    assert c != b
    huge = alloc((64 << 20) + 1)
    assert lib.cuda_free(huge) == 0 and lib.cuda_free(c) == 0
    base = lib.mx_metadata_table_size()
    meta = np.arange(8, dtype=np.uint64)
    assert lib.cuda_memcpy_h2d(b + 4096, meta.ctypes.data, meta.nbytes) == 0      # recorded, keyed by an interior address
    assert lib.mx_metadata_table_size() == base + 1
    big = np.zeros(1024, dtype=np.uint64)
    assert lib.cuda_memcpy_h2d(b + 4096 - 64, big.ctypes.data, big.nbytes) == 0   # too large to record; overlaps the entry
    assert lib.mx_metadata_table_size() == base
    assert lib.cuda_memcpy_h2d(b + 8192, meta.ctypes.data, meta.nbytes) == 0
    assert lib.mx_metadata_table_size() == base + 1
    assert lib.cuda_free(b) == 0                                                   # frees the whole 128 KB block
    assert lib.mx_metadata_table_size() == base


@pytest.mark.parametrize("dt", [D.F32, D.BF16, D.F16, D.F64, D.U8, D.I32, D.I64], ids=lambda d: d.name)
def test_flat_operands_at_unaligned_offsets(oracle, cuda, dt):
    """Contiguous operands whose first element is not on a 16-byte boundary (every fixture of the reference's own tests
    is a view from element 1) run on the shifted form of the flat kernel: every offset class, different offsets for
    the two inputs, lengths around the vector and block sizes, a bool-valued comparison and an in-place update."""
    rng = np.random.default_rng(zlib.crc32(dt.name.encode()))
    vec = 16 // dt.size
    for n in (1, vec - 1, vec, vec + 1, 5 * vec + 3, 4096 + 5, 100003):
        for loff, roff in ((1, 1), (1, 0), (3, 2), (vec - 1, vec + 1), (0, 5)):
            a = H.random_store(rng, dt, n + loff + 3, lo=-50, hi=50) if dt.kind != "float" else H.random_store(rng, dt, n + loff + 3)
            b = H.random_store(rng, dt, n + roff + 3, lo=1, hi=50) if dt.kind != "float" else H.random_store(rng, dt, n + roff + 3, lo=0.5, hi=2.0)
            for op in ("add", "div", "lt"):
                args = (op, dt, [n], [1], [1], loff, roff, a, b)
                H.assert_same(op, dt, H.run_binary(cuda, *args), H.run_binary(oracle, *args), what=f"n={n} offsets=({loff},{roff})")
            args = ("mul_inplace", dt, [n], [1], [1], loff, roff, a, b)
            H.assert_same("mul_inplace", dt, H.run_binary_inplace(cuda, *args), H.run_binary_inplace(oracle, *args), what=f"inplace n={n} ({loff},{roff})")
        got = H.run_unary(cuda, "neg" if dt.kind != "uint" else "square", dt, [n], [1], 1, a)
        ref = H.run_unary(oracle, "neg" if dt.kind != "uint" else "square", dt, [n], [1], 1, a)
        H.assert_same("unary", dt, got, ref, what=f"unary n={n}")
    # a 2-d dense view at offset 1 merges to the same flat form; a scalar rhs (stride 0) stays a broadcast
    a, b = H.random_store(rng, dt, 64 * 70 + 1), H.random_store(rng, dt, 2)
    args = ("add", dt, [64, 70], [70, 1], [0, 0], 1, 1, a, b)
    H.assert_same("add", dt, H.run_binary(cuda, *args), H.run_binary(oracle, *args), what="2-d + scalar")


@pytest.mark.parametrize("dt", [D.BF16, D.F16, D.I16, D.U16], ids=lambda d: d.name)
def test_two_byte_transposed_tiles(oracle, cuda, dt):
    """2-byte types with vector-aligned transposed operands run on the tensor-copy tile kernel (64 x 64 boxes, ldmatrix
    transposition): ragged edges in both dims, padded pitches, aligned base offsets, one batch dim (also broadcast for
    one operand), and the layouts that kernel hands back to the general one (two batch dims, a stride-0 direct operand)."""
    rng = np.random.default_rng(zlib.crc32(dt.name.encode()) + 16)
    P, Q = 200, 136
    cases = [
        ("ragged", [P, Q], [1, P], [Q, 1], 0, 0, P * Q, P * Q),
        ("ragged-both-transposed", [P, Q], [1, P], [1, P], 8, 16, P * Q + 8, P * Q + 16),
        ("padded-pitches", [P, Q], [1, P + 24], [Q + 8, 1], 0, 8, (P + 24) * Q, (Q + 8) * P + 8),
        ("rhs-transposed", [72, 328], [328, 1], [1, 72], 0, 0, 72 * 328, 72 * 328),
        ("batched", [5, 72, 136], [72 * 136, 1, 72], [72 * 136, 136, 1], 0, 0, 5 * 72 * 136, 5 * 72 * 136),
        ("batch-broadcast-rhs", [5, 72, 136], [72 * 136, 1, 72], [0, 136, 1], 0, 0, 5 * 72 * 136, 72 * 136),
        ("two-batch-dims", [2, 3, 72, 136], [3 * 72 * 136, 72 * 136, 1, 72], [0, 72 * 136, 136, 1], 0, 0, 6 * 72 * 136, 3 * 72 * 136),
        ("row-broadcast-rhs", [P, Q], [1, P], [0, 1], 0, 0, P * Q, Q),
        ("single-tile", [64, 64], [1, 64], [64, 1], 0, 0, 4096, 4096),
        ("small", [8, 16], [1, 8], [16, 1], 0, 0, 128, 128),
    ]
    for name, dims, ls, rs, lo, ro, ll, rl in cases:
        if dt.kind == "float":
            lhs, rhs = H.random_store(rng, dt, ll), H.random_store(rng, dt, rl, lo=0.5, hi=2.0)
        else:
            lhs, rhs = H.random_store(rng, dt, ll, lo=0 if dt.kind == "uint" else -90, hi=90), H.random_store(rng, dt, rl, lo=1, hi=90)
        for op in ("add", "div", "maximum"):
            args = (op, dt, dims, ls, rs, lo, ro, lhs, rhs)
            H.assert_same(op, dt, H.run_binary(cuda, *args), H.run_binary(oracle, *args), what=name)
        uop = "square" if dt.kind == "uint" else "neg"
        H.assert_same(uop, dt, H.run_unary(cuda, uop, dt, dims, ls, lo, lhs), H.run_unary(oracle, uop, dt, dims, ls, lo, lhs), what=f"unary {name}")


def test_wait_report_of_a_staged_kernel_is_surfaced_by_the_next_copy(oracle, cuda):
    """The kernels that are fed through shared memory by the copy engine (staged flat operands, 2-byte transposed tiles,
    staged col2im) record a bounded wait that ran out in the same per-device word as the tensor-core products, with
    codes 21..23.  The ABI's own synchronisation points report it.  The word is written from the host - no wait has to
    run out on the GPU - and the launch made over the stale report still computes its result."""
    import ctypes
    from maidenx_b200 import _lib, device
    lib = _lib.load()
    poke = lib.mx_debug_tc_gemm_poke_status
    poke.argtypes, poke.restype = [ctypes.c_int], ctypes.c_int
    dt = D.BF16
    rng = np.random.default_rng(5)
    P, Q = 128, 192
    lhs, rhs = H.random_store(rng, dt, P * Q), H.random_store(rng, dt, P * Q)
    ref = H.run_binary(oracle, "add", dt, [P, Q], [1, P], [Q, 1], 0, 0, lhs, rhs)
    assert poke(22) == 0
    bufs = [device.CudaBuffer.from_host(x) for x in (lhs, rhs, np.zeros(P * Q, dt.np_storage))]
    try:
        meta = [P, Q, 1, P, Q, 1, 0, 0]
        device.dispatch("add", dt.name, meta, ctypes.c_size_t(P * Q), ctypes.c_size_t(2), "META", bufs[0].ptr, bufs[1].ptr, bufs[2].ptr)
        out = np.empty(P * Q, dt.np_storage)
        rc = lib.cuda_memcpy_d2h(out.ctypes.data, bufs[2].ptr, out.nbytes)
        assert rc != 0, "the copy that follows the op must report the device-side wait"
        assert lib.mx_last_error() == 5 and lib.mx_last_cuda_error() == 22
        assert b"staged" in lib.mx_last_error_where()
        lib.mx_clear_error()
        H.assert_same("add", dt, out, ref, what="tile op launched over a stale report")
        assert lib.cuda_memcpy_d2h(out.ctypes.data, bufs[2].ptr, out.nbytes) == 0  # reported once, then clear
    finally:
        lib.mx_clear_error()
        for x in bufs:
            x.free()
