// General batched matmul on the CUDA cores: every dtype, every stride pattern, and the
// index quirks of the reference (the parity target is crates/maidenx_cpu/src/ops/matmul.rs).
// The tensor-core path (matmul_tc.cu) takes over for bf16 / f16 shapes it supports; this
// kernel is the fallback and the only path for f32 / f64 / integers.
//
// One kernel serves forward and both backward products.  It computes
//     out[row * N + col] = sum_{r < K} X[ix(row, r)] * Y[iy(row, r, col)]
// with affine index functions, row = batch * M + mi:
//     ix = batch * xs_b + mi * xs_m + r * xs_r        (term skipped when ix >= x_limit)
//     iy = batch * ys_b + r * ys_r + col * ys_c       (term skipped when iy >= y_limit)
// which covers C = A.B with contiguous or strided operands (matmul.rs:74-113),
// grad_a = g.B^T (:196-219) and grad_b = A^T.g (:231-261), whose loops read A, B and g as
// contiguous whatever their strides, and the bounds checks those loops carry.
//
// Accumulation order is k ascending inside one thread, so results are reproducible and:
// integers are exact (wrapping), f32 / f64 match the reference's element-type accumulation
// bit for bit (no FMA contraction), bf16 / f16 accumulate in f32 and round once.
#pragma once
#include "common.cuh"
#include "ops.cuh"

namespace mx {

struct MmParams {
    uint64_t rows;      // number of output rows (batch * M, or ceil(out_elems / N))
    uint64_t N, K;      // output columns, reduction length
    uint64_t M;         // rows per batch
    uint64_t out_elems; // elements of out that may be written (last row may be short)
    int64_t xs_b, xs_m, xs_r;
    int64_t ys_b, ys_r, ys_c;
    uint64_t x_limit, y_limit;
};

template <class T>
struct MmAcc {
    typedef typename std::conditional<is_half_v<T>, f32,
            typename std::conditional<is_fp_v<T>, T,
            typename std::conditional<sizeof(T) == 8, u64, u32>::type>::type>::type type;
};
template <class T>
__device__ __forceinline__ typename MmAcc<T>::type mm_load(T v) {
    if constexpr (is_half_v<T>) return to_f32(v);
    else return (typename MmAcc<T>::type)v;
}
template <class T>
__device__ __forceinline__ T mm_store(typename MmAcc<T>::type a) {
    if constexpr (is_half_v<T>) return from_f32<T>(a);
    else return (T)a;
}

constexpr int kMmTile = 64;   // output tile edge
constexpr int kMmK = 16;      // reduction step
constexpr int kMmThreads = 256;

template <class T>
__global__ void __launch_bounds__(kMmThreads) matmul_simt_kernel(const T* __restrict__ X, const T* __restrict__ Y, T* __restrict__ out, MmParams P) {
    typedef typename MmAcc<T>::type Acc;
    __shared__ Acc xs[kMmK][kMmTile + 1];  // [r][row]
    __shared__ Acc ys[kMmK][kMmTile + 1];  // [r][col]
    const uint64_t row0 = (uint64_t)blockIdx.x * kMmTile, col0 = (uint64_t)blockIdx.y * kMmTile;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
    Acc acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = (Acc)0;

    // loader mapping: pick the fast index along the operand's smaller stride
    const bool x_r_fast = (P.xs_r <= P.xs_m) || P.xs_m == 0;
    const bool y_c_fast = (P.ys_c <= P.ys_r) || P.ys_r == 0;

    for (uint64_t k0 = 0; k0 < P.K; k0 += kMmK) {
#pragma unroll
        for (int it = 0; it < (kMmTile * kMmK) / kMmThreads; it++) {
            int e = threadIdx.x + it * kMmThreads;
            int lr, lrow;
            if (x_r_fast) {
                lr = e % kMmK;
                lrow = e / kMmK;
            } else {
                lrow = e % kMmTile;
                lr = e / kMmTile;
            }
            uint64_t row = row0 + lrow, r = k0 + lr;
            Acc v = (Acc)0;
            if (row < P.rows && r < P.K) {
                uint64_t batch = row / P.M, mi = row % P.M;
                uint64_t ix = (uint64_t)((int64_t)batch * P.xs_b + (int64_t)mi * P.xs_m + (int64_t)r * P.xs_r);
                if (ix < P.x_limit) v = mm_load<T>(X[ix]);
            }
            xs[lr][lrow] = v;
        }
#pragma unroll
        for (int it = 0; it < (kMmTile * kMmK) / kMmThreads; it++) {
            int e = threadIdx.x + it * kMmThreads;
            int lr, lcol;
            if (y_c_fast) {
                lcol = e % kMmTile;
                lr = e / kMmTile;
            } else {
                lr = e % kMmK;
                lcol = e / kMmK;
            }
            // the batch of a tile row is needed for Y too; rows of one tile may span batches,
            // so Y is staged per (r, col) for the batch of the tile's FIRST row and re-read
            // directly for rows of other batches (rare: only when M is not a multiple of 64)
            uint64_t col = col0 + lcol, r = k0 + lr;
            Acc v = (Acc)0;
            if (col < P.N && r < P.K) {
                uint64_t batch = row0 / P.M;
                uint64_t iy = (uint64_t)((int64_t)batch * P.ys_b + (int64_t)r * P.ys_r + (int64_t)col * P.ys_c);
                if (iy < P.y_limit) v = mm_load<T>(Y[iy]);
            }
            ys[lr][lcol] = v;
        }
        __syncthreads();
        const uint64_t batch0 = row0 / P.M;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint64_t row = row0 + ty * 4 + i;
            if (row >= P.rows) continue;
            uint64_t batch = row / P.M;
            if (batch == batch0) {
#pragma unroll
                for (int kk = 0; kk < kMmK; kk++) {
                    Acc xv = xs[kk][ty * 4 + i];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if constexpr (is_half_v<T>) acc[i][j] = fmaf(xv, ys[kk][tx * 4 + j], acc[i][j]);  // product exact in f32
                        else acc[i][j] = acc[i][j] + xv * ys[kk][tx * 4 + j];
                    }
                }
            } else {
                // this row belongs to a later batch than the staged Y tile: read Y directly
                for (int kk = 0; kk < kMmK; kk++) {
                    uint64_t r = k0 + kk;
                    if (r >= P.K) break;
                    Acc xv = xs[kk][ty * 4 + i];
                    for (int j = 0; j < 4; j++) {
                        uint64_t col = col0 + tx * 4 + j;
                        Acc yv = (Acc)0;
                        if (col < P.N) {
                            uint64_t iy = (uint64_t)((int64_t)batch * P.ys_b + (int64_t)r * P.ys_r + (int64_t)col * P.ys_c);
                            if (iy < P.y_limit) yv = mm_load<T>(Y[iy]);
                        }
                        if constexpr (is_half_v<T>) acc[i][j] = fmaf(xv, yv, acc[i][j]);
                        else acc[i][j] = acc[i][j] + xv * yv;
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint64_t row = row0 + ty * 4 + i;
        if (row >= P.rows) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint64_t col = col0 + tx * 4 + j;
            uint64_t o = row * P.N + col;
            if (col < P.N && o < P.out_elems) out[o] = mm_store<T>(acc[i][j]);
        }
    }
}

// Few outputs, long reduction (the weight gradient of a narrow Linear layer: [1, batch] . [batch, in] in the reference's
// README example): the tiled kernel would run the whole reduction in one or two blocks.  Here one block owns one output
// element, its threads take k = t, t + 256, ... (each in ascending order) and the partial sums are folded by a fixed
// shuffle tree, so the result is reproducible; integers stay exact (wrapping addition is associative), floats are summed
// in a different order than the element-type loop of the reference and agree with it within the reduction tolerance.
template <class T>
__global__ void __launch_bounds__(kMmThreads) matmul_longk_kernel(const T* __restrict__ X, const T* __restrict__ Y, T* __restrict__ out, MmParams P) {
    typedef typename MmAcc<T>::type Acc;
    const uint64_t o = blockIdx.x;
    const uint64_t row = o / P.N, col = o % P.N;
    const uint64_t batch = row / P.M, mi = row % P.M;
    const int64_t x0 = (int64_t)batch * P.xs_b + (int64_t)mi * P.xs_m, y0 = (int64_t)batch * P.ys_b + (int64_t)col * P.ys_c;
    Acc acc = (Acc)0;
    for (uint64_t r = threadIdx.x; r < P.K; r += kMmThreads) {
        const uint64_t ix = (uint64_t)(x0 + (int64_t)r * P.xs_r), iy = (uint64_t)(y0 + (int64_t)r * P.ys_r);
        const Acc xv = ix < P.x_limit ? mm_load<T>(X[ix]) : (Acc)0, yv = iy < P.y_limit ? mm_load<T>(Y[iy]) : (Acc)0;
        if constexpr (is_half_v<T>) acc = fmaf(xv, yv, acc);
        else acc = acc + xv * yv;
    }
    __shared__ Acc part[kMmThreads / 32];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc = acc + __shfl_down_sync(0xFFFFFFFFu, acc, s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        Acc total = part[0];
#pragma unroll
        for (int w = 1; w < kMmThreads / 32; w++) total = total + part[w];
        if (o < P.out_elems) out[o] = mm_store<T>(total);
    }
}
constexpr uint64_t kLongKMinK = 2048, kLongKMaxOutputs = 1024;

// Host-side description of one matmul call, parsed from the metadata block
// [out_ndim, a_ndim, b_ndim | out_shape | a_shape | b_shape | a_strides | b_strides | a_off, b_off]
// (crates/maidenx_tensor/src/ops/matmul.rs:227-264).
struct MmDesc {
    bool valid;
    size_t out_nd, a_nd, b_nd;
    uint64_t m, n, k_fwd, k_bwd;
    uint64_t g_size;               // product of out_shape (1 when out_ndim == 0)
    bool a_cont, b_cont;
    int64_t a_strides[3];          // batch (a_strides[0]), row (a_strides[nd-2]), col (a_strides[nd-1]); rank 1: col only
    int64_t b_strides[3];
    uint64_t a_off, b_off;
};
bool mm_parse(const size_t* hm, MmDesc& d);
size_t mm_meta_words(const size_t* head3);

template <class T>
void mm_launch(const MmParams& P, const T* X, const T* Y, T* out, const char* where) {
    if (P.rows == 0 || P.N == 0) return;
    if (P.K >= kLongKMinK && P.out_elems <= kLongKMaxOutputs && P.rows * P.N <= kLongKMaxOutputs) {
        matmul_longk_kernel<T><<<(unsigned)P.out_elems, kMmThreads, 0, ctx().stream>>>(X, Y, out, P);
        check_launch(where);
        return;
    }
    uint64_t gx = (P.rows + kMmTile - 1) / kMmTile, gy = (P.N + kMmTile - 1) / kMmTile;
    if (gy > 65535 || gx > 0x7FFFFFFFull) {  // more than 4M output columns
        set_error(kErrUnsupported, 0, where);
        return;
    }
    dim3 grid((unsigned)gx, (unsigned)gy);
    matmul_simt_kernel<T><<<grid, kMmThreads, 0, ctx().stream>>>(X, Y, out, P);
    check_launch(where);
}

}  // namespace mx
