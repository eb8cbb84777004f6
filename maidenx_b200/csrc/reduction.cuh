// Reductions: sum / mean / max / min along dims and sum_to_shape (the broadcast-gradient
// fold of backward).
//
// The reference scatters every input element into out[fold(i)] with one global atomic per
// element (crates/maidenx_cuda/kernels/ops/reduction.cu:18-63) or one mutex acquisition
// (crates/maidenx_cpu/src/ops/reduction.rs:45-58).  Here the host recognises the
// contiguous [outer O, reduced R, inner I] structure and runs one of:
//   rows    (I == 1) each row of R contiguous elements is reduced by a thread, a warp or
//           a block (by length) with 16-byte loads and a warp-shuffle tree; when there are
//           too few rows to fill the GPU each row is split over several blocks;
//   cols    (I > 1) each thread owns a 16-byte strip of columns and walks down R; R is split
//           over blockIdx.y so that a [8192,16384] -> [16384] fold still fills 148 SMs;
// split reductions write per-block partials to scratch and a second launch folds them:
// the classic two-pass grid reduce.  Every path is atomic-free, so results are
// deterministic, and the output is overwritten (no pre-zero contract).
// Accumulation: bf16/f16 in f32 with one final rounding, f32 in f32, f64 in f64, integers
// wrapping in 32/64 bits (truncation to the element width commutes with wrapping adds).
// Anything else (several reduced dims, non-contiguous input, partial sum_to_shape
// factors) follows the reference's index formulas literally through a scatter kernel with
// wide atomics into scratch.
#pragma once
#include <cfloat>

#include "common.cuh"
#include "ops.cuh"

namespace mx {

enum RedKind { RED_SUM = 0, RED_MEAN = 1, RED_MAX = 2, RED_MIN = 3 };

// ---------------------------------------------------------------------------------
// accumulator traits
// ---------------------------------------------------------------------------------
template <class T, int KIND>
struct RedTraits;

template <class T>
struct SumAcc {
    typedef typename std::conditional<is_half_v<T>, f32,
            typename std::conditional<is_fp_v<T>, T,
            typename std::conditional<sizeof(T) == 8, u64, u32>::type>::type>::type type;
};
template <class T>
struct MaxAcc {
    typedef typename std::conditional<is_half_v<T>, f32,
            typename std::conditional<is_fp_v<T>, T,
            typename std::conditional<sizeof(T) == 8, T,
            typename std::conditional<std::is_signed<T>::value, i32, u32>::type>::type>::type>::type type;
};

template <class T, int KIND>
struct RedTraits {
    static constexpr bool kIsSum = KIND == RED_SUM || KIND == RED_MEAN;
    typedef typename std::conditional<kIsSum, typename SumAcc<T>::type, typename MaxAcc<T>::type>::type Acc;

    __host__ __device__ static Acc init() {
        if constexpr (kIsSum) return (Acc)0;
        else if constexpr (KIND == RED_MAX) {
            // crates/maidenx_cpu/src/ops/reduction.rs:603-614: T::MIN; for 16-bit floats f32::MIN rounds to -inf
            if constexpr (is_half_v<T>) return -INFINITY;
            else if constexpr (std::is_same<T, f32>::value) return -FLT_MAX;
            else if constexpr (std::is_same<T, f64>::value) return -DBL_MAX;
            else return (Acc)std::numeric_limits<T>::min();
        } else {
            if constexpr (is_half_v<T>) return INFINITY;
            else if constexpr (std::is_same<T, f32>::value) return FLT_MAX;
            else if constexpr (std::is_same<T, f64>::value) return DBL_MAX;
            else return (Acc)std::numeric_limits<T>::max();
        }
    }
    __device__ __forceinline__ static Acc load(T v) {
        if constexpr (is_half_v<T>) return to_f32(v);
        else return (Acc)v;  // integers: sign- or zero-extended, then wrapped in Acc
    }
    __device__ __forceinline__ static Acc combine(Acc a, Acc v) {
        // max / min: a NaN never wins (the reference's `if val > *out`), whichever side of a
        // pairwise combine it arrives on.
        if constexpr (kIsSum) return a + v;
        else if constexpr (std::is_same<Acc, f32>::value) {
            // the hardware max / min return the other operand when one is NaN, and the initial
            // value is never NaN, so a NaN can only survive a combine of two NaNs and then loses
            // the next one: the same outcome as the reference's comparison, in one instruction
            if constexpr (KIND == RED_MAX) return fmaxf(a, v);
            else return fminf(a, v);
        } else if constexpr (std::is_same<Acc, f64>::value) {
            if constexpr (KIND == RED_MAX) return fmax(a, v);
            else return fmin(a, v);
        } else if constexpr (KIND == RED_MAX) return v > a ? v : a;
        else return v < a ? v : a;
    }
    // factor: number of reduced elements (mean only)
    __device__ __forceinline__ static T finalize(Acc a, u64 factor) {
        if constexpr (KIND == RED_MEAN) {
            // the reference divides the finished sum by the count converted to the element type
            if constexpr (is_half_v<T>) return from_f32<T>(a / to_f32(from_f32<T>((f32)factor)));
            else return (T)(a / (Acc)(T)factor);
        } else if constexpr (is_half_v<T>) return from_f32<T>(a);
        else return (T)a;
    }
};

// ---------------------------------------------------------------------------------
// block / warp reduce
// ---------------------------------------------------------------------------------
template <class TR>
__device__ __forceinline__ typename TR::Acc warp_reduce(typename TR::Acc v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = TR::combine(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
template <class TR, int THREADS>
__device__ __forceinline__ typename TR::Acc block_reduce(typename TR::Acc v) {
    __shared__ typename TR::Acc warp_part[THREADS / 32];
    v = warp_reduce<TR>(v);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    v = threadIdx.x < THREADS / 32 ? warp_part[threadIdx.x] : TR::init();
    if (threadIdx.x < 32) v = warp_reduce<TR>(v);
    return v;  // valid in thread 0
}

constexpr int kRedThreads = 256;

// ---------------------------------------------------------------------------------
// rows: in[row * R + r], out[row]
// ---------------------------------------------------------------------------------
// One block per (row, split).  grid = (splits, rows).  VEC > 1 requires R % VEC == 0,
// seg % VEC == 0 and a 16-byte aligned base.
template <class T, int KIND, int VEC, class Src, class SrcTR>
__device__ __forceinline__ typename SrcTR::Acc row_segment(const Src* row, u64 begin, u64 end) {
    typedef typename SrcTR::Acc Acc;
    Acc acc0 = SrcTR::init(), acc1 = SrcTR::init(), acc2 = SrcTR::init(), acc3 = SrcTR::init();
    const u64 step = (u64)kRedThreads * VEC;
    u64 i = begin + (u64)threadIdx.x * VEC;
    // four independent vector loads in flight per thread
    for (; i + 3 * step < end; i += 4 * step) {
        Vec<Src, VEC> a = *reinterpret_cast<const Vec<Src, VEC>*>(row + i);
        Vec<Src, VEC> b = *reinterpret_cast<const Vec<Src, VEC>*>(row + i + step);
        Vec<Src, VEC> c = *reinterpret_cast<const Vec<Src, VEC>*>(row + i + 2 * step);
        Vec<Src, VEC> d = *reinterpret_cast<const Vec<Src, VEC>*>(row + i + 3 * step);
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            acc0 = SrcTR::combine(acc0, SrcTR::load(a.v[j]));
            acc1 = SrcTR::combine(acc1, SrcTR::load(b.v[j]));
            acc2 = SrcTR::combine(acc2, SrcTR::load(c.v[j]));
            acc3 = SrcTR::combine(acc3, SrcTR::load(d.v[j]));
        }
    }
    for (; i < end; i += step) {
        Vec<Src, VEC> a = *reinterpret_cast<const Vec<Src, VEC>*>(row + i);
#pragma unroll
        for (int j = 0; j < VEC; j++) acc0 = SrcTR::combine(acc0, SrcTR::load(a.v[j]));
    }
    return SrcTR::combine(SrcTR::combine(acc0, acc1), SrcTR::combine(acc2, acc3));
}

// Arrival counting for split reductions that fold their partials in the same launch: every block
// publishes its partial (write, __threadfence), then one thread bumps the counter of its output
// group; the block that sees the last ticket re-reads all partials of the group, folds them in
// split order (so the result does not depend on which block came last) and writes the output.
// It also puts the counter back to zero, so the counter array is all-zero between launches.
__device__ __forceinline__ bool last_arrival(u32* counter, u32 expected) {
    __shared__ u32 s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const u32 ticket = atomicAdd(counter, 1u);
        s_last = ticket == expected - 1;
        if (s_last) *counter = 0;
    }
    __syncthreads();
    const bool last = s_last != 0;
    if (last) __threadfence();
    return last;
}
template <class Acc>
__device__ __forceinline__ Acc load_published(const Acc* p) {
    return *reinterpret_cast<const volatile Acc*>(p);  // not through L1: written by other blocks of this launch
}

// counters == nullptr: partials are left for a second launch (reduce_partials_*_kernel).
template <class T, int KIND, int VEC>
__global__ void __launch_bounds__(kRedThreads) reduce_rows_block_kernel(const T* in, T* out, typename RedTraits<T, KIND>::Acc* partial,
                                                                      u64 R, u64 seg, u32 splits, u64 factor, u32* counters, int tree_fold) {
    typedef RedTraits<T, KIND> TR;
    typedef typename TR::Acc Acc;
    const u64 row = blockIdx.y;
    const u32 split = blockIdx.x;
    const u64 begin = (u64)split * seg;
    u64 end = begin + seg;
    if (end > R) end = R;
    Acc v = begin < end ? row_segment<T, KIND, VEC, T, TR>(in + row * R, begin, end) : TR::init();
    v = block_reduce<TR, kRedThreads>(v);
    if (threadIdx.x == 0) {
        if (splits == 1) out[row] = TR::finalize(v, factor);
        else partial[row * splits + split] = v;
    }
    if (splits == 1 || !counters) return;
    if (!last_arrival(counters + row, splits)) return;
    const Acc* mine = partial + row * splits;
    if (tree_fold) {  // same shape as reduce_partials_block_kernel
        Acc acc = TR::init();
        for (u32 s2 = threadIdx.x; s2 < splits; s2 += kRedThreads) acc = TR::combine(acc, load_published(mine + s2));
        acc = block_reduce<TR, kRedThreads>(acc);
        if (threadIdx.x == 0) out[row] = TR::finalize(acc, factor);
    } else if (threadIdx.x == 0) {  // same order as reduce_partials_kernel
        Acc acc = TR::init();
        for (u32 s2 = 0; s2 < splits; s2++) acc = TR::combine(acc, load_published(mine + s2));
        out[row] = TR::finalize(acc, factor);
    }
}

// One warp per row (32 <= R < ~2048).
template <class T, int KIND, int VEC>
__global__ void __launch_bounds__(kRedThreads) reduce_rows_warp_kernel(const T* in, T* out, u64 rows, u64 R, u64 factor) {
    typedef RedTraits<T, KIND> TR;
    const u64 row = (u64)blockIdx.x * (kRedThreads / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* p = in + row * R;
    typename TR::Acc acc = TR::init();
    for (u64 i = (u64)lane * VEC; i < R; i += 32 * VEC) {
        Vec<T, VEC> a = *reinterpret_cast<const Vec<T, VEC>*>(p + i);
#pragma unroll
        for (int j = 0; j < VEC; j++) acc = TR::combine(acc, TR::load(a.v[j]));
    }
    acc = warp_reduce<TR>(acc);
    if (lane == 0) out[row] = TR::finalize(acc, factor);
}

// One thread per row (R < 32).
template <class T, int KIND>
__global__ void __launch_bounds__(kRedThreads) reduce_rows_thread_kernel(const T* in, T* out, u64 rows, u64 R, u64 factor) {
    typedef RedTraits<T, KIND> TR;
    const u64 row = (u64)blockIdx.x * kRedThreads + threadIdx.x;
    if (row >= rows) return;
    const T* p = in + row * R;
    typename TR::Acc acc = TR::init();
    for (u64 i = 0; i < R; i++) acc = TR::combine(acc, TR::load(p[i]));
    out[row] = TR::finalize(acc, factor);
}

// Second pass of a split reduction: out[j] = fold of partial[j * S + s] (rows layout) or
// partial[s * count + j] (cols layout).  One thread per output.
template <class T, int KIND>
__global__ void __launch_bounds__(kRedThreads) reduce_partials_kernel(const typename RedTraits<T, KIND>::Acc* partial, T* out, u64 count,
                                                                    u32 S, int cols_layout, u64 factor) {
    typedef RedTraits<T, KIND> TR;
    const u64 j = (u64)blockIdx.x * kRedThreads + threadIdx.x;
    if (j >= count) return;
    typename TR::Acc acc = TR::init();
    if (cols_layout) {
        for (u32 s = 0; s < S; s++) acc = TR::combine(acc, partial[(u64)s * count + j]);
    } else {
        for (u32 s = 0; s < S; s++) acc = TR::combine(acc, partial[j * S + s]);
    }
    out[j] = TR::finalize(acc, factor);
}

// Same fold with one block per output, for few outputs with many partials (a full reduction
// split over ~1000 blocks): threads stride over the partials, then a fixed-shape block tree.
template <class T, int KIND>
__global__ void __launch_bounds__(kRedThreads) reduce_partials_block_kernel(const typename RedTraits<T, KIND>::Acc* partial, T* out, u32 S, u64 factor) {
    typedef RedTraits<T, KIND> TR;
    const u64 j = blockIdx.x;
    typename TR::Acc acc = TR::init();
    for (u32 s = threadIdx.x; s < S; s += kRedThreads) acc = TR::combine(acc, partial[j * S + s]);
    acc = block_reduce<TR, kRedThreads>(acc);
    if (threadIdx.x == 0) out[j] = TR::finalize(acc, factor);
}

// ---------------------------------------------------------------------------------
// cols: in[(o * R + r) * I + i], out[o * I + i]
// ---------------------------------------------------------------------------------
constexpr int kColLanes = 32;  // threads along the columns
constexpr int kColRows = 8;    // threads along the reduced dim

// grid = (ceil(I / (32 * VEC)), splits, min(O, 65535)).  VEC > 1 requires I % VEC == 0 and an
// aligned base.
template <class T, int KIND, int VEC>
__global__ void __launch_bounds__(kColLanes* kColRows) reduce_cols_kernel(const T* in, T* out, typename RedTraits<T, KIND>::Acc* partial, u64 O,
                                                                         u64 R, u64 I, u64 seg, u32 splits, u64 factor, u32* counters) {
    typedef RedTraits<T, KIND> TR;
    typedef typename TR::Acc Acc;
    __shared__ Acc sm[kColRows][kColLanes * VEC + 1];
    const int lane = threadIdx.x % kColLanes, ty = threadIdx.x / kColLanes;
    const u64 col = ((u64)blockIdx.x * kColLanes + lane) * VEC;
    const u32 split = blockIdx.y;
    const u64 r_begin = (u64)split * seg;
    u64 r_end = r_begin + seg;
    if (r_end > R) r_end = R;
    for (u64 o = blockIdx.z; o < O; o += gridDim.z) {
        Acc acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; j++) acc[j] = TR::init();
        if (col < I) {
            const T* p = in + o * R * I + col;
            u64 r = r_begin + ty;
            // eight independent 16-byte loads in flight per thread
            for (; r + 7 * kColRows < r_end; r += 8 * kColRows) {
                Vec<T, VEC> x[8];
#pragma unroll
                for (int q = 0; q < 8; q++) x[q] = *reinterpret_cast<const Vec<T, VEC>*>(p + (r + q * kColRows) * I);
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    Acc s01 = TR::combine(TR::load(x[0].v[j]), TR::load(x[1].v[j]));
                    Acc s23 = TR::combine(TR::load(x[2].v[j]), TR::load(x[3].v[j]));
                    Acc s45 = TR::combine(TR::load(x[4].v[j]), TR::load(x[5].v[j]));
                    Acc s67 = TR::combine(TR::load(x[6].v[j]), TR::load(x[7].v[j]));
                    acc[j] = TR::combine(acc[j], TR::combine(TR::combine(s01, s23), TR::combine(s45, s67)));
                }
            }
            for (; r < r_end; r += kColRows) {
                Vec<T, VEC> a = *reinterpret_cast<const Vec<T, VEC>*>(p + r * I);
#pragma unroll
                for (int j = 0; j < VEC; j++) acc[j] = TR::combine(acc[j], TR::load(a.v[j]));
            }
        }
#pragma unroll
        for (int j = 0; j < VEC; j++) sm[ty][lane * VEC + j] = acc[j];
        __syncthreads();
        // fold the kColRows partial strips; the first kColLanes*VEC threads each own a column
        for (int c = threadIdx.x; c < kColLanes * VEC; c += kColLanes * kColRows) {
            u64 gc = (u64)blockIdx.x * kColLanes * VEC + c;
            if (gc < I) {
                Acc v = sm[0][c];
#pragma unroll
                for (int y = 1; y < kColRows; y++) v = TR::combine(v, sm[y][c]);
                if (splits == 1) out[o * I + gc] = TR::finalize(v, factor);
                else partial[((u64)split * O + o) * I + gc] = v;
            }
        }
        if (splits > 1 && counters) {
            // fold in the same launch: the last block of this (o, column strip) to arrive
            if (last_arrival(counters + o * gridDim.x + blockIdx.x, splits)) {
                for (int c = threadIdx.x; c < kColLanes * VEC; c += kColLanes * kColRows) {
                    u64 gc = (u64)blockIdx.x * kColLanes * VEC + c;
                    if (gc < I) {
                        Acc v = TR::init();
                        for (u32 s2 = 0; s2 < splits; s2++) v = TR::combine(v, load_published(partial + ((u64)s2 * O + o) * I + gc));
                        out[o * I + gc] = TR::finalize(v, factor);
                    }
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------
// generic scatter path (literal index formulas, wide atomics into scratch)
// ---------------------------------------------------------------------------------
constexpr int kRedMaxDims = 16;

struct RedGenParams {
    int mode;  // 0 = dim reduction, 1 = sum_to_shape
    u64 n;
    int nd, nr;
    int contiguous;
    u64 dims[kRedMaxDims], strides[kRedMaxDims];
    u64 red_len[kRedMaxDims], red_stride[kRedMaxDims];  // mode 0
    u64 out_dims[kRedMaxDims];                         // mode 1
    u64 off;
};

template <class Acc>
__device__ __forceinline__ void atomic_combine_sum(Acc* p, Acc v) {
    if constexpr (std::is_same<Acc, u64>::value) atomicAdd(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
    else atomicAdd(p, v);
}
template <class Acc, bool IS_MAX>
__device__ __forceinline__ void atomic_combine_minmax(Acc* p, Acc v) {
    if constexpr (std::is_same<Acc, f32>::value || std::is_same<Acc, f64>::value) {
        typedef typename std::conditional<sizeof(Acc) == 4, unsigned int, unsigned long long>::type Bits;
        Bits* bp = reinterpret_cast<Bits*>(p);
        Bits old = *bp;
        for (int guard = 0; guard < (1 << 20); guard++) {
            Acc cur;
            memcpy(&cur, &old, sizeof(Acc));
            bool better = IS_MAX ? (v > cur) : (v < cur);
            if (!better) return;
            Bits nb;
            memcpy(&nb, &v, sizeof(Acc));
            Bits prev = atomicCAS(bp, old, nb);
            if (prev == old) return;
            old = prev;
        }
    } else if constexpr (std::is_same<Acc, i64>::value) {
        if (IS_MAX) atomicMax(reinterpret_cast<long long*>(p), (long long)v);
        else atomicMin(reinterpret_cast<long long*>(p), (long long)v);
    } else if constexpr (std::is_same<Acc, u64>::value) {
        if (IS_MAX) atomicMax(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
        else atomicMin(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
    } else {
        if (IS_MAX) atomicMax(p, v);
        else atomicMin(p, v);
    }
}

template <class T, int KIND>
__global__ void __launch_bounds__(kRedThreads) reduce_fill_kernel(typename RedTraits<T, KIND>::Acc* ws, u64 count) {
    for (u64 j = (u64)blockIdx.x * kRedThreads + threadIdx.x; j < count; j += (u64)gridDim.x * kRedThreads) ws[j] = RedTraits<T, KIND>::init();
}
template <class T, int KIND>
__global__ void __launch_bounds__(kRedThreads) reduce_finalize_kernel(const typename RedTraits<T, KIND>::Acc* ws, T* out, u64 count, u64 factor) {
    for (u64 j = (u64)blockIdx.x * kRedThreads + threadIdx.x; j < count; j += (u64)gridDim.x * kRedThreads)
        out[j] = RedTraits<T, KIND>::finalize(ws[j], factor);
}

template <class T, int KIND>
__global__ void __launch_bounds__(kRedThreads) reduce_scatter_kernel(const T* in, typename RedTraits<T, KIND>::Acc* ws, RedGenParams P) {
    typedef RedTraits<T, KIND> TR;
    for (u64 i = (u64)blockIdx.x * kRedThreads + threadIdx.x; i < P.n; i += (u64)gridDim.x * kRedThreads) {
        u64 src, dst;
        if (P.mode == 0) {
            // crates/maidenx_cpu/src/ops/reduction.rs:45-79
            src = i;
            if (!P.contiguous) {
                u64 rem = i;
                src = 0;
                for (int d = P.nd - 1; d >= 0; d--) {
                    if (P.strides[d] != 0) src += (rem % P.dims[d]) * P.strides[d];
                    rem /= P.dims[d];
                }
            }
            dst = i;
            for (int k = 0; k < P.nr; k++) {
                u64 s = P.red_stride[k], l = P.red_len[k];
                if (s != 0) {
                    u64 pre = dst / s, post = dst % s;
                    dst = (pre / l) * s + post;
                } else {
                    dst /= l;
                }
            }
        } else {
            // crates/maidenx_cpu/src/ops/reduction.rs:127-170
            u64 rem = i, lin = 0, mul = 1;
            src = 0;
            // walk dims from the innermost: coordinate, strided source, row-major index in out_dims
            for (int d = P.nd - 1; d >= 0; d--) {
                u64 c = rem % P.dims[d];
                rem /= P.dims[d];
                src += c * P.strides[d];
                u64 f = P.dims[d] / P.out_dims[d];
                lin += (c / f) * mul;
                mul *= P.out_dims[d];
            }
            dst = lin;
            if (P.contiguous) src = i;
            else src = (src + P.off) % P.n;  // the reference adds the offset a second time and wraps
        }
        typename TR::Acc v = TR::load(in[src]);
        if constexpr (TR::kIsSum) atomic_combine_sum(ws + dst, v);
        else atomic_combine_minmax<typename TR::Acc, KIND == RED_MAX>(ws + dst, v);
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
enum RedPlanKind { RP_EMPTY = 0, RP_ROWS, RP_COLS, RP_GENERIC, RP_ERROR };

struct RedPlan {
    int kind;
    u64 O, R, I;      // rows: O rows of R; cols: [O, R, I]
    u64 out_count;
    u64 factor;       // elements folded into each output (mean divisor)
    u64 off;
    RedGenParams gen;
};

// How many ways to split each of `groups` independent reductions so that the launch fills the
// GPU's `capacity` resident blocks in ONE wave: a launch of slightly more blocks than fit pays a
// second, nearly empty wave, which on these 50-100 us kernels costs 10-20 %.
inline u64 split_count(u64 groups, u64 capacity) {
    if (groups == 0 || groups >= capacity) return 1;
    u64 s = capacity / groups;
    return s < 1 ? 1 : s;
}
u32* arrival_counters(u64 count);                      // zeroed counters for last_arrival, or nullptr if count is too large

void red_plan_dims(RedPlan& pl, size_t num_els, size_t num_dims, size_t num_red, const size_t* hm);
void red_plan_shape(RedPlan& pl, size_t num_els, size_t num_dims, const size_t* hm);

template <class T, int KIND>
void red_launch(const RedPlan& pl, const T* in, T* out, const char* where) {
    typedef RedTraits<T, KIND> TR;
    typedef typename TR::Acc Acc;
    constexpr int VEC = 16 / sizeof(T);
    cudaStream_t s = ctx().stream;
    const int sms = sm_count();
    if (pl.kind == RP_EMPTY) return;
    if (pl.kind == RP_ERROR) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    in += pl.off;
    const bool base_aligned = ((uintptr_t)in) % 16 == 0;
    if (pl.kind == RP_ROWS) {
        const u64 O = pl.O, R = pl.R;
        if (R < 32) {
            u64 blocks = (O + kRedThreads - 1) / kRedThreads;
            reduce_rows_thread_kernel<T, KIND><<<(u32)blocks, kRedThreads, 0, s>>>(in, out, O, R, pl.factor);
        } else if (R < 2048 && O >= (u64)sms * 4) {
            u64 blocks = (O + 7) / 8;
            if (base_aligned && R % VEC == 0) reduce_rows_warp_kernel<T, KIND, VEC><<<(u32)blocks, kRedThreads, 0, s>>>(in, out, O, R, pl.factor);
            else reduce_rows_warp_kernel<T, KIND, 1><<<(u32)blocks, kRedThreads, 0, s>>>(in, out, O, R, pl.factor);
        } else {
            // block per (row, split); split long rows when there are too few rows to fill the GPU
            const bool vec = base_aligned && R % VEC == 0;
            const u64 unit = (u64)kRedThreads * VEC * 4;  // one full unrolled trip of a block
            static int occ = 0;  // resident blocks per SM of this instantiation
            if (!occ) occ = resident_blocks((const void*)reduce_rows_block_kernel<T, KIND, VEC>, kRedThreads);
            u64 want = split_count(O, (u64)sms * occ);
            u64 max_splits = (R + unit - 1) / unit;
            u64 splits = want < max_splits ? want : max_splits;
            if (splits < 1) splits = 1;
            u64 seg = (R + splits - 1) / splits;
            seg = (seg + VEC - 1) / VEC * VEC;
            splits = (R + seg - 1) / seg;
            if (O > 65535) {  // grid.y limit: fall back to one warp per row
                u64 blocks = (O + 7) / 8;
                reduce_rows_warp_kernel<T, KIND, 1><<<(u32)blocks, kRedThreads, 0, s>>>(in, out, O, R, pl.factor);
            } else {
                Acc* part = nullptr;
                u32* counters = nullptr;
                if (splits > 1) {
                    part = static_cast<Acc*>(scratch(sizeof(Acc) * O * splits));
                    if (!part) return;
                    counters = arrival_counters(O);  // nullptr: too many groups, fold in a second launch
                }
                const int tree_fold = O <= 64 && splits >= 64;
                dim3 grid((u32)splits, (u32)O);
                if (vec) reduce_rows_block_kernel<T, KIND, VEC><<<grid, kRedThreads, 0, s>>>(in, out, part, R, seg, (u32)splits, pl.factor, counters, tree_fold);
                else reduce_rows_block_kernel<T, KIND, 1><<<grid, kRedThreads, 0, s>>>(in, out, part, R, seg, (u32)splits, pl.factor, counters, tree_fold);
                if (splits > 1 && !counters) {
                    check_launch(where);
                    if (tree_fold) reduce_partials_block_kernel<T, KIND><<<(u32)O, kRedThreads, 0, s>>>(part, out, (u32)splits, pl.factor);
                    else reduce_partials_kernel<T, KIND><<<(u32)((O + kRedThreads - 1) / kRedThreads), kRedThreads, 0, s>>>(part, out, O, (u32)splits, 0, pl.factor);
                }
            }
        }
        check_launch(where);
        return;
    }
    if (pl.kind == RP_COLS) {
        const u64 O = pl.O, R = pl.R, I = pl.I;
        const bool vec = base_aligned && I % VEC == 0;
        const int v = vec ? VEC : 1;
        u64 gx = (I + (u64)kColLanes * v - 1) / ((u64)kColLanes * v);
        u64 gz = O < 65535 ? O : 65535;
        static int occ = 0;
        if (!occ) occ = resident_blocks((const void*)reduce_cols_kernel<T, KIND, VEC>, kColLanes * kColRows);
        u64 want = split_count(gx * gz, (u64)sms * occ);
        u64 max_splits = (R + 63) / 64;  // at least 64 rows per split
        u64 splits = want < max_splits ? want : max_splits;
        if (splits < 1) splits = 1;
        if (splits > 65535) splits = 65535;
        u64 seg = (R + splits - 1) / splits;
        splits = (R + seg - 1) / seg;
        Acc* part = nullptr;
        u32* counters = nullptr;
        if (splits > 1) {
            part = static_cast<Acc*>(scratch(sizeof(Acc) * splits * O * I));
            if (!part) return;
            counters = arrival_counters(O * gx);
        }
        dim3 grid((u32)gx, (u32)splits, (u32)gz);
        if (vec) reduce_cols_kernel<T, KIND, VEC><<<grid, kColLanes * kColRows, 0, s>>>(in, out, part, O, R, I, seg, (u32)splits, pl.factor, counters);
        else reduce_cols_kernel<T, KIND, 1><<<grid, kColLanes * kColRows, 0, s>>>(in, out, part, O, R, I, seg, (u32)splits, pl.factor, counters);
        if (splits > 1 && !counters) {
            check_launch(where);
            u64 count = O * I;
            reduce_partials_kernel<T, KIND><<<(u32)((count + kRedThreads - 1) / kRedThreads), kRedThreads, 0, s>>>(part, out, count, (u32)splits, 1, pl.factor);
        }
        check_launch(where);
        return;
    }
    // generic scatter
    Acc* ws = static_cast<Acc*>(scratch(sizeof(Acc) * (pl.out_count ? pl.out_count : 1)));
    if (!ws) return;
    u32 fill_blocks = (u32)((pl.out_count + kRedThreads - 1) / kRedThreads);
    if (fill_blocks > (u32)sms * 16) fill_blocks = sms * 16;
    if (fill_blocks == 0) fill_blocks = 1;
    reduce_fill_kernel<T, KIND><<<fill_blocks, kRedThreads, 0, s>>>(ws, pl.out_count);
    u64 sb = (pl.gen.n + kRedThreads - 1) / kRedThreads;
    if (sb > (u64)sms * 16) sb = (u64)sms * 16;
    if (sb) reduce_scatter_kernel<T, KIND><<<(u32)sb, kRedThreads, 0, s>>>(in, ws, pl.gen);
    reduce_finalize_kernel<T, KIND><<<fill_blocks, kRedThreads, 0, s>>>(ws, out, pl.out_count, pl.factor);
    check_launch(where);
}

template <class T, int KIND>
void reduce_entry(size_t n, size_t nd, size_t nr, const size_t* meta, const T* in, T* out, const char* where) {
    const size_t* hm = resolve_metadata(meta, 2 * nd + 2 * nr + 1);
    if (!hm) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    RedPlan pl;
    red_plan_dims(pl, n, nd, nr, hm);
    red_launch<T, KIND>(pl, in, out, where);
}
template <class T>
void sum_to_shape_entry(size_t n, size_t nd, const size_t* meta, const T* in, T* out, const char* where) {
    const size_t* hm = resolve_metadata(meta, 3 * nd + 1);
    if (!hm) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    RedPlan pl;
    red_plan_shape(pl, n, nd, hm);
    red_launch<T, RED_SUM>(pl, in, out, where);
}

}  // namespace mx
