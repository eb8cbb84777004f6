"""The host-side launch planners, without a GPU: layouts of the benchmark and of the parity tests must be
recognised as the kernel class that was written for them (a silent fall to the generic gather kernel would keep
every parity test green and lose an order of magnitude of bandwidth)."""
import ctypes

import numpy as np

from maidenx_b200 import _lib

FLAT, ROW, TILE, GENERIC, SERIAL, FLAT_SHIFT = 1, 2, 3, 4, 5, 7
ROWS, COLS, SCATTER = 1, 2, 3
BASE = 0x7F0000000000  # a 256-byte aligned pretend device address: the planner only looks at alignment


def ew_plan(meta, nd, n, nin=2, inplace=False, esz=4, osz=4, out=BASE, a=BASE + (1 << 32), b=BASE + (2 << 32)):
    lib = _lib.load()
    m = np.asarray(meta, dtype=np.uint64)
    rank, vec, tmask = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    kind = lib.mx_debug_elementwise_plan(n, nd, m.ctypes.data, nin, int(inplace), esz, osz, out, a, b, ctypes.byref(rank), ctypes.byref(vec),
                                         ctypes.byref(tmask))
    return kind, rank.value, vec.value, tmask.value


def test_benchmark_layouts_take_their_kernels():
    R = C = 16384
    n = R * C
    assert ew_plan([R, C, C, 1, C, 1, 0, 0], 2, n)[:3] == (FLAT, 1, 1)                 # contiguous: merged to one dim
    kind, rank, vec, tmask = ew_plan([R, C, 1, R, C, 1, 0, 0], 2, n)                    # transposed lhs
    assert (kind, vec, tmask) == (TILE, 1, 1)
    assert ew_plan([R, C, C, 1, 0, 1, 0, 0], 2, n)[:3] == (ROW, 2, 1)                  # rhs broadcast from [1, C]
    assert ew_plan([R, C, 1, R, 0], 2, n, nin=1)[0] == TILE                            # unary on a transposed view
    assert ew_plan([R, C, 0, 1, 0], 2, n, nin=1)[0] == ROW                             # unary on a broadcast row
    for esz in (2, 4, 8):
        assert ew_plan([R, C, 1, R, C, 1, 0, 0], 2, n, esz=esz, osz=esz)[0] == TILE


def test_odd_layouts_degrade_gracefully():
    # offset 1 (the layout of the reference's test fixtures) breaks 16-byte alignment: the call takes the flat kernel's
    # shifted form (aligned 16-byte loads + funnel shift), not the per-element gather
    assert ew_plan([1000, 1, 1, 1, 1], 1, 1000)[:3] == (FLAT_SHIFT, 1, 1)
    # the same view at an aligned offset is flat again
    assert ew_plan([1000, 1, 1, 4, 8], 1, 1000)[:3] == (FLAT, 1, 1)
    # a permuted 3-d view has no unit-stride pairing the tile kernel handles
    assert ew_plan([5, 6, 7, 1, 35, 5, 42, 7, 1, 0, 0], 3, 210)[0] == GENERIC
    # size-1 dims are dropped before anything else
    assert ew_plan([1, 9, 1, 11, 99, 11, 11, 1, 99, 11, 11, 1, 0, 0], 4, 99)[:2] == (FLAT, 1)
    # both operands transposed the same way: the output is the only direct operand
    kind, _, _, tmask = ew_plan([96, 80, 1, 96, 1, 96, 0, 0], 2, 96 * 80)
    assert (kind, tmask) == (TILE, 3)
    # in-place with an lhs that overlaps itself (stride 0) must run serially
    assert ew_plan([8, 4, 0, 1, 4, 1, 0, 0], 2, 32, inplace=True, out=BASE, a=BASE)[0] == SERIAL
    # scalars
    assert ew_plan([2, 1], 0, 1)[0] in (FLAT, GENERIC)


def red_plan(meta, nd, nr, n, shape=False):
    lib = _lib.load()
    m = np.asarray(meta, dtype=np.uint64)
    o, r, i = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_size_t()
    kind = lib.mx_debug_reduce_plan(n, nd, nr, m.ctypes.data, int(shape), ctypes.byref(o), ctypes.byref(r), ctypes.byref(i))
    return kind, o.value, r.value, i.value


def test_reduction_layouts_take_their_kernels():
    R, C = 8192, 16384
    n = R * C
    assert red_plan([R, C, C, 1, R, C, 0], 2, 1, n) == (COLS, 1, R, C)                  # dim 0: fold 8192 rows of 16384 columns
    assert red_plan([R, C, C, 1, C, 1, 0], 2, 1, n)[:3] == (ROWS, R, C)                 # dim 1: 8192 rows of 16384
    # sum_to_shape [64, 512, 4096] -> [1, 1, 4096]: the two leading dims fold into one reduced extent
    assert red_plan([64, 512, 4096, 512 * 4096, 4096, 1, 1, 1, 4096, 0], 3, 0, 64 * 512 * 4096, shape=True) == (COLS, 1, 64 * 512, 4096)
    # the middle dim of a 3-d tensor
    assert red_plan([7, 129, 5, 645, 5, 1, 129, 5, 0], 3, 1, 7 * 129 * 5) == (COLS, 7, 129, 5)
    # a full reduction as the MLP's bias gradient issues it
    assert red_plan([1 << 20, 1, 1 << 20, 1, 0], 1, 1, 1 << 20)[:3] == (ROWS, 1, 1 << 20)
    # two reduced dims at once, or a transposed input, follow the reference's index formulas literally
    assert red_plan([4, 6, 8, 48, 8, 1, 4, 8, 48, 1, 0], 3, 2, 192)[0] == SCATTER
    assert red_plan([64, 32, 1, 64, 64, 1, 0], 2, 1, 2048)[0] == SCATTER


def mm_path(meta, num_els, a=BASE, b=BASE + (1 << 32), out=BASE + (2 << 32), f32=False):
    lib = _lib.load()
    m_ = np.asarray(meta, dtype=np.uint64)
    amn, bmn = ctypes.c_int(-1), ctypes.c_int(-1)
    M, N, K = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_size_t()
    fn = lib.mx_debug_matmul_forward_path_f32 if f32 else lib.mx_debug_matmul_forward_path
    tc = fn(num_els, m_.ctypes.data, a, b, out, ctypes.byref(amn), ctypes.byref(bmn), ctypes.byref(M),
                                          ctypes.byref(N), ctypes.byref(K))
    return tc, amn.value, bmn.value, M.value, N.value, K.value


def test_the_three_products_of_a_linear_layer_run_on_the_tensor_core_kernel():
    """Forward x . W^T (B read through a transposed view), dW = du^T . a (A through a transposed view) and
    dX = du . W (both dense), at the benchmark's per-rank shapes for 1 and 8 ranks: none needs a transposed copy."""
    D = 8192
    for B in (16384, 2048):
        assert mm_path([2, 2, 2, B, D, B, D, D, D, D, 1, 1, D, 0, 0], B * D) == (1, 0, 0, B, D, D)       # NT: both K-major
        assert mm_path([2, 2, 2, D, D, D, B, B, D, 1, D, D, 1, 0, 0], D * D) == (1, 1, 1, D, D, B)       # TN: both MN-major
        assert mm_path([2, 2, 2, B, D, B, D, D, D, D, 1, D, 1, 0, 0], B * D) == (1, 0, 1, B, D, D)       # NN


def test_products_the_tensor_core_kernel_does_not_take():
    assert mm_path([2, 2, 2, 64, 64, 64, 64, 64, 64, 64, 1, 64, 1, 0, 0], 64 * 64)[0] == 0               # too small for a persistent launch
    assert mm_path([2, 2, 2, 512, 516, 512, 512, 512, 516, 512, 1, 516, 1, 0, 0], 512 * 516)[0] == 0     # N not a multiple of 8 elements
    assert mm_path([2, 2, 2, 512, 512, 512, 512, 512, 512, 512, 1, 512, 1, 1, 0], 512 * 512)[0] == 0     # offset 1: base not 16-byte aligned
    assert mm_path([2, 2, 2, 512, 512, 512, 512, 512, 512, 1024, 2, 512, 1, 0, 0], 512 * 512)[0] == 0    # A with a stride of 2 along k
    assert mm_path([3, 3, 3, 4, 512, 512, 4, 512, 512, 4, 512, 512, 262144, 512, 1, 262144, 512, 1, 0, 0], 4 * 512 * 512)[0] == 4  # batched rank-3: one launch, four batches
    assert mm_path([4, 4, 4, 2, 2, 512, 512, 2, 2, 512, 512, 2, 2, 512, 512, 524288, 262144, 512, 1, 524288, 262144, 512, 1, 0, 0], 4 * 512 * 512)[0] == 0  # rank 4


def test_f32_products_take_the_split_tf32_kernel_when_rows_are_16_byte_multiples():
    """f32: the contiguous extent of each matrix must be a multiple of 4 elements (16 bytes for TMA), not 8."""
    D = 8192
    assert mm_path([2, 2, 2, 2048, D, 2048, D, D, D, D, 1, 1, D, 0, 0], 2048 * D, f32=True) == (1, 0, 0, 2048, D, D)
    # conv forward at the benchmark shape: cols [200704, 2304] . weight^T view of [256, 2304]
    assert mm_path([2, 2, 2, 200704, 256, 200704, 2304, 2304, 256, 2304, 1, 1, 2304, 0, 0], 200704 * 256, f32=True) == (1, 0, 0, 200704, 256, 2304)
    assert mm_path([2, 2, 2, 512, 516, 512, 512, 512, 516, 512, 1, 516, 1, 0, 0], 512 * 516, f32=True)[0] == 1   # 516 = 4 * 129
    assert mm_path([2, 2, 2, 512, 514, 512, 512, 512, 514, 512, 1, 514, 1, 0, 0], 512 * 514, f32=True)[0] == 0
    assert mm_path([2, 2, 2, 64, 64, 64, 64, 64, 64, 64, 1, 64, 1, 0, 0], 64 * 64, f32=True)[0] == 0             # small: SIMT, bit-exact order


def test_split_k_plan():
    """Few output tiles and a long reduction are cut along K so that every SM gets a tile; products that already fill
    the GPU, short reductions and K that does not divide are left alone."""
    lib = _lib.load()
    sk = lib.mx_debug_splitk_slices
    assert sk(18, 200704, 64, 148) == 8          # the conv weight gradient at the benchmark shape: 144 tiles on 148 SMs
    assert sk(36, 200704, 32, 148) == 4          # the same product in f32 (128 x 128 tiles)
    assert sk(4096, 8192, 64, 148) == 1          # the MLP products fill the GPU
    assert sk(4, 2048, 64, 148) == 1             # reduction too short to be worth a second pass
    assert sk(2, 65600, 64, 148) == 1 or 65600 % (64 * sk(2, 65600, 64, 148)) == 0
    for tiles, k in ((1, 1 << 20), (3, 65536), (10, 16384)):
        s_ = sk(tiles, k, 64, 148)
        assert s_ >= 1 and (k // 64) % s_ == 0 and k // s_ >= 1024


def test_b_panel_resident_schedule_is_for_short_reductions_with_many_row_tiles():
    lib = _lib.load()
    keep = lib.mx_debug_gemm_keep_b_ctas
    assert keep(1568, 9, 4, 1, 148) == 16      # the conv input-gradient product (200704 x 2304 x 256): 16 CTAs per column tile
    assert keep(1568, 9, 5, 1, 148) == 0       # K = 320 does not fit the four-slot ring
    assert keep(1568, 9, 4, 2, 148) == 0       # batched products keep the general schedule
    assert keep(40, 9, 4, 1, 148) == 0         # too few row tiles per CTA to spread the panel's load over
    assert keep(1568, 200, 4, 1, 148) == 0     # more column tiles than CTAs
    assert keep(400, 1, 2, 1, 148) == 0        # 148 CTAs on one column tile: fewer than four row tiles each
    assert keep(1000, 1, 2, 1, 148) == 148
