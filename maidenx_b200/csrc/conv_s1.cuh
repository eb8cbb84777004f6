// Stride-1 fast paths of im2col / col2im (the 3x3 / pad 1 convolution of the benchmark and any
// kw in {1,3,5,7} with "same" or no horizontal padding).  The general kernels in conv.cu spend
// their time on per-element index arithmetic and 2-byte accesses; here every thread moves whole
// 16-byte vectors and the kw shift is a compile-time selection out of two neighbouring vectors.
//
// im2col: the (b,c) plane is staged in shared memory WITH its zero border, so a work item is
// "one padded input row x one output vector": it reads the 16-byte window that covers all kw
// shifts once and stores kw vectors for each of the kh output rows that row feeds.
// col2im: a work item is one output vector of a row; for every (kh, kw) it loads the two aligned
// col vectors that cover its shifted window and accumulates in the reference's order
// (kh descending = h_out ascending, kw descending = w_out ascending) and in the element type.
#pragma once
#include "common.cuh"
#include "ops.cuh"
#include "tc_ptx.cuh"

namespace mx {

struct ConvS1Params {
    uint32_t H, W, KH, OH, OW, PH, PW;
    uint32_t pitch;      // elements per staged row (im2col)
    uint32_t owv;        // output vectors per row = OW / VEC
    uint64_t num_els;    // readable length of col (col2im)
};

constexpr int kConvS1Threads = 256;

// element j of the 2*VEC-element window held in two vectors
template <class T, int VEC>
__device__ __forceinline__ T window_at(const Vec<T, VEC>& lo, const Vec<T, VEC>& hi, int j) {
    return j < VEC ? lo.v[j] : hi.v[j - VEC];
}

template <class T, int VEC, int KW>
__global__ void __launch_bounds__(kConvS1Threads) im2col_s1_kernel(const T* __restrict__ x, T* __restrict__ col, ConvS1Params P) {
    extern __shared__ __align__(16) unsigned char conv_s1_smem[];
    T* plane = reinterpret_cast<T*>(conv_s1_smem);
    const uint64_t bc = blockIdx.x;
    const uint32_t rows_p = P.H + 2 * P.PH;
    const T zero = zero_of<T>();
    // zero border + payload
    for (uint32_t i = threadIdx.x; i < rows_p * P.pitch; i += kConvS1Threads) plane[i] = zero;
    __syncthreads();
    const T* src = x + bc * (uint64_t)P.H * P.W;
    for (uint32_t i = threadIdx.x; i < P.H * P.W; i += kConvS1Threads) {
        uint32_t h = i / P.W, w = i - h * P.W;
        plane[(h + P.PH) * P.pitch + P.PW + w] = src[i];
    }
    __syncthreads();
    const uint32_t OHW = P.OH * P.OW;
    T* dst_plane = col + bc * (uint64_t)P.KH * KW * OHW;
    const uint32_t items = rows_p * P.owv;
    for (uint32_t it = threadIdx.x; it < items; it += kConvS1Threads) {
        const uint32_t hp = it / P.owv, ov = it - hp * P.owv;
        const T* row = plane + hp * P.pitch + ov * VEC;
        const Vec<T, VEC> lo = *reinterpret_cast<const Vec<T, VEC>*>(row);
        const Vec<T, VEC> hi = *reinterpret_cast<const Vec<T, VEC>*>(row + VEC);
        Vec<T, VEC> shifted[KW];
#pragma unroll
        for (int kw = 0; kw < KW; kw++)
#pragma unroll
            for (int j = 0; j < VEC; j++) shifted[kw].v[j] = window_at<T, VEC>(lo, hi, kw + j);
        // padded row hp feeds output row ho = hp - kh of kernel row kh
        for (uint32_t kh = 0; kh < P.KH; kh++) {
            if (hp < kh) break;
            const uint32_t ho = hp - kh;
            if (ho >= P.OH) continue;
            T* d = dst_plane + (uint64_t)kh * KW * OHW + (uint64_t)ho * P.OW + ov * VEC;
#pragma unroll
            for (int kw = 0; kw < KW; kw++) *reinterpret_cast<Vec<T, VEC>*>(d + (uint64_t)kw * OHW) = shifted[kw];
        }
    }
}

template <class T>
__device__ __forceinline__ T conv_s1_add(T a, T b) {
    if constexpr (is_half_v<T>) return from_f32<T>(to_f32(a) + to_f32(b));
    else return a + b;
}

// One (kh, kw) term for all VEC pixels of the item.  KWI and PW are template parameters so that
// the window shift PW - KWI is a compile-time constant; the recursion walks kw from KW-1 down to 0
// (w_out ascending).
template <class T, int VEC, int KW, int PW, int KWI>
__device__ __forceinline__ void col2im_s1_terms(const T* __restrict__ col, const ConvS1Params& P, uint64_t kh_base, uint32_t w0, uint32_t OHW,
                                                const Vec<T, VEC>& zero_vec, Vec<T, VEC>& sum) {
    // pixel w0 + j reads col column w0 + j + SH
    constexpr int SH = PW - KWI;                          // |SH| < VEC on this path
    constexpr int E = ((SH % VEC) + VEC) % VEC;           // offset inside the first aligned vector
    const int a0 = (int)w0 + (SH >= 0 ? 0 : -VEC);        // column of the first aligned vector
    const uint64_t row_base = kh_base + (uint64_t)KWI * OHW;
    Vec<T, VEC> lo = zero_vec, hi = zero_vec;
    if (a0 >= 0 && (uint32_t)a0 < P.OW && row_base + a0 + VEC <= P.num_els) lo = *reinterpret_cast<const Vec<T, VEC>*>(col + row_base + a0);
    if (E != 0 && a0 + VEC >= 0 && (uint32_t)(a0 + VEC) < P.OW && row_base + a0 + 2 * VEC <= P.num_els)
        hi = *reinterpret_cast<const Vec<T, VEC>*>(col + row_base + a0 + VEC);
    Vec<T, VEC> term;
#pragma unroll
    for (int j = 0; j < VEC; j++) term.v[j] = window_at<T, VEC>(lo, hi, E + j);
    if constexpr (is_half_v<T>) {
        // packed 16-bit adds round exactly like "add in f32, round" (see HalfNative in ops.cuh)
        uint32_t* sw = reinterpret_cast<uint32_t*>(&sum);
        const uint32_t* tw = reinterpret_cast<const uint32_t*>(&term);
#pragma unroll
        for (int j = 0; j < VEC / 2; j++) sw[j] = HalfNative<OpAdd>::template f<T>(sw[j], tw[j]);
    } else {
#pragma unroll
        for (int j = 0; j < VEC; j++) sum.v[j] = conv_s1_add(sum.v[j], term.v[j]);
    }
    if constexpr (KWI > 0) col2im_s1_terms<T, VEC, KW, PW, KWI - 1>(col, P, kh_base, w0, OHW, zero_vec, sum);
}

template <class T, int VEC, int KW, int PW>
__global__ void __launch_bounds__(kConvS1Threads) col2im_s1_kernel(const T* __restrict__ col, T* __restrict__ out, ConvS1Params P) {
    const uint64_t bc = blockIdx.y;
    const uint32_t wv = P.W / VEC;  // output vectors per image row (W % VEC == 0 on this path)
    const uint32_t item = blockIdx.x * kConvS1Threads + threadIdx.x;
    if (item >= P.H * wv) return;
    const uint32_t h = item / wv, w0 = (item - h * wv) * VEC;
    const uint32_t hp = h + P.PH;
    const uint32_t OHW = P.OH * P.OW;
    const uint64_t plane_base = bc * (uint64_t)P.KH * KW * OHW;
    Vec<T, VEC> sum;
#pragma unroll
    for (int j = 0; j < VEC; j++) sum.v[j] = zero_of<T>();
    const Vec<T, VEC> zero_vec = sum;
    // h_out ascending = kh descending
    for (int kh = (int)min(P.KH - 1, hp); kh >= 0; kh--) {
        const uint32_t ho = hp - kh;
        if (ho >= P.OH) continue;
        const uint64_t kh_base = plane_base + (uint64_t)kh * KW * OHW + (uint64_t)ho * P.OW;
        col2im_s1_terms<T, VEC, KW, PW, KW - 1>(col, P, kh_base, w0, OHW, zero_vec, sum);
    }
    *reinterpret_cast<Vec<T, VEC>*>(out + bc * (uint64_t)P.H * P.W + (uint64_t)h * P.W + w0) = sum;
}

// col2im with the block's column planes staged in shared memory: one block per (b, c) plane asks the SM's copy engine
// (cp.async.bulk, completion on an mbarrier, bounded wait) for the KH * KW consecutive [OH, OW] planes that feed it - every
// column entry crosses from L2 once, in full lines - and the shifted windows are then cut out of shared memory by the same
// term walk as above (same order, same rounding).  Needs the whole column buffer readable (num_els covers every plane) and
// KH * KW * OH * OW elements to fit the shared memory of at least two resident blocks.
template <class T, int VEC, int KW, int PW>
__global__ void __launch_bounds__(kConvS1Threads) col2im_s1_staged_kernel(const T* __restrict__ col, T* __restrict__ out, ConvS1Params P, tc::WaitReport rep) {
    extern __shared__ __align__(128) unsigned char conv_s1_stage[];
    __shared__ __align__(8) unsigned long long stage_bar;
    const T* planes = reinterpret_cast<const T*>(conv_s1_stage);
    const uint64_t bc = blockIdx.x;
    const uint32_t OHW = P.OH * P.OW;
    const uint32_t plane_elems = P.KH * KW * OHW;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&stage_bar);
    if (threadIdx.x == 0) {
        const uint32_t bytes = plane_elems * (uint32_t)sizeof(T);
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         (uint32_t)__cvta_generic_to_shared(conv_s1_stage)),
                     "l"(col + bc * (uint64_t)plane_elems), "r"(bytes), "r"(bar)
                     : "memory");
    }
    __syncthreads();
    bool landed = false;
    for (int i = 0; i < (1 << 26) && !landed; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar)
            : "memory");
        landed = ok != 0;
    }
    if (!landed) {
        tc::wait_gave_up(rep, 23);  // surfaces as status 5 at the caller's next synchronisation point
        return;
    }
    ConvS1Params L = P;
    L.num_els = plane_elems;  // everything staged is readable
    const uint32_t wv = P.W / VEC;
    Vec<T, VEC> zero_vec;
#pragma unroll
    for (int j = 0; j < VEC; j++) zero_vec.v[j] = zero_of<T>();
    for (uint32_t item = threadIdx.x; item < P.H * wv; item += kConvS1Threads) {
        const uint32_t h = item / wv, w0 = (item - h * wv) * VEC;
        const uint32_t hp = h + P.PH;
        Vec<T, VEC> sum = zero_vec;
        for (int kh = (int)min(P.KH - 1, hp); kh >= 0; kh--) {
            const uint32_t ho = hp - kh;
            if (ho >= P.OH) continue;
            const uint64_t kh_base = (uint64_t)kh * KW * OHW + (uint64_t)ho * P.OW;
            col2im_s1_terms<T, VEC, KW, PW, KW - 1>(planes, L, kh_base, w0, OHW, zero_vec, sum);
        }
        *reinterpret_cast<Vec<T, VEC>*>(out + bc * (uint64_t)P.H * P.W + (uint64_t)h * P.W + w0) = sum;
    }
}

}  // namespace mx
