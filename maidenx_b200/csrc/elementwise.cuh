// Strided elementwise engine shared by the binary, in-place binary, unary and
// unary-with-constant families.
//
// The host reduces the (dims, strides, offsets) metadata of the C ABI to a canonical
// form — size-1 dims dropped, adjacent dims merged wherever every operand allows it —
// and picks one of four kernels:
//   flat     every operand is one contiguous run (or a broadcast scalar): 16-byte
//            vector loads/stores, four vectors in flight per thread;
//   row      every operand has stride 1 or 0 along the innermost dim; outer dims are
//            arbitrary (row-vector / column-vector broadcasts, padded rows): one
//            fast-divmod per 16-byte vector instead of per element;
//   tile     an input is unit-stride along another dim (a transposed view): 64x64
//            tiles staged through shared memory so both the transposed read and the
//            output write are full 128-byte lines;
//   shifted  flat operands whose addresses are not 16-byte aligned (the offset-1 views of the reference's test
//            fixtures): a scalar head brings the output to a 16-byte boundary, then every input vector is
//            assembled from the two aligned 16-byte words it straddles with a funnel shift;
//   generic  anything else: per-element fast-divmod gather.
// In-place ops reuse the same kernels with the output aliased to the lhs and the dims
// re-ordered by the lhs strides; an lhs that overlaps itself (stride 0) runs serially
// on one thread, which is the order the CPU backend applies.
#pragma once
#include "common.cuh"
#include "ops.cuh"
#include "tc_ptx.cuh"

namespace mx {

enum EwKind { EW_EMPTY = 0, EW_FLAT, EW_ROW, EW_TILE, EW_GENERIC, EW_SERIAL, EW_ERROR, EW_FLAT_SHIFT };

struct EwPlan {
    int kind;
    int nin;
    uint64_t n;
    int nd;
    uint32_t dim[kMaxDims];
    int64_t st[3][kMaxDims];  // element strides: 0 = out, 1 = a, 2 = b
    int64_t off[3];           // element offsets applied to the base pointers
    int p;                    // tile: the dim along which the transposed inputs are unit-stride
    bool transposed[3];       // tile: operand is read through shared memory
    bool vec;                 // 16-byte vector access is legal for every operand
};

// in_size / out_size: element sizes in bytes; ptrs: base addresses (out, a, b) before offsets.
void ew_make_plan(EwPlan& pl, size_t num_els, size_t num_dims, const size_t* hmeta, int nin, bool inplace, size_t in_size,
                  size_t out_size, const void* out, const void* a, const void* b);

// ---------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------
constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;

template <class T, int N>
__device__ __forceinline__ Vec<T, N> ld_vec(const T* p) {
    return *reinterpret_cast<const Vec<T, N>*>(p);
}
template <class T, int N>
__device__ __forceinline__ void st_vec(T* p, const Vec<T, N>& v) {
    *reinterpret_cast<Vec<T, N>*>(p) = v;
}
template <class T, int N>
__device__ __forceinline__ Vec<T, N> splat(T x) {
    Vec<T, N> v;
#pragma unroll
    for (int i = 0; i < N; i++) v.v[i] = x;
    return v;
}

template <class F, class T, class O, int NIN, int VEC>
__device__ __forceinline__ Vec<O, VEC> apply_vec(const F& f, const Vec<T, VEC>& a, const Vec<T, VEC>& b) {
    Vec<O, VEC> r;
    if constexpr (F::kNative && VEC % 2 == 0 && NIN == 2) {
        // bf16 / f16 add and sub: the packed hardware instruction rounds exactly as "f32, then round"
        const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
        const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
        uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
        for (int i = 0; i < VEC / 2; i++) rw[i] = f.native(aw[i], bw[i]);
    } else if constexpr (F::kChecked && VEC % 2 == 0) {
        // bf16 / f16 division: approximate quotients, and the few elements the check flags are
        // redone with the exact out-of-line division
        const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
        const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
        uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
        uint32_t mask = 0;
#pragma unroll
        for (int i = 0; i < VEC / 2; i++) {
            float2 x = unpack2<T>(aw[i]);
            if constexpr (NIN == 2) {
                float2 y = unpack2<T>(bw[i]);
                rw[i] = pack2_rn<T>(f.core_checked(x.x, y.x, mask, 2 * i), f.core_checked(x.y, y.y, mask, 2 * i + 1));
            } else {
                rw[i] = pack2_rn<T>(f.core_checked(x.x, mask, 2 * i), f.core_checked(x.y, mask, 2 * i + 1));
            }
        }
        if (mask) {
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                if ((mask >> i) & 1u) {
                    if constexpr (NIN == 2) r.v[i] = f(a.v[i], b.v[i]);
                    else r.v[i] = f(a.v[i]);
                }
            }
        }
    } else if constexpr (F::kCore && VEC % 2 == 0) {
        // 16-bit floats: unpack / compute in f32 / round two elements at a time
        const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
        const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
        uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
        for (int i = 0; i < VEC / 2; i++) {
            float2 x = unpack2<T>(aw[i]);
            if constexpr (NIN == 2) {
                float2 y = unpack2<T>(bw[i]);
                rw[i] = pack2_rn<T>(f.core(x.x, y.x), f.core(x.y, y.y));
            } else {
                rw[i] = pack2_rn<T>(f.core(x.x), f.core(x.y));
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; i++) {
            if constexpr (NIN == 2) r.v[i] = f(a.v[i], b.v[i]);
            else r.v[i] = f(a.v[i]);
        }
    }
    return r;
}

// sa / sb: 1 = contiguous, 0 = broadcast scalar
template <class F, class T, class O, int NIN, int VEC>
__global__ void __launch_bounds__(kEwThreads) ew_flat_kernel(F f, const T* a, const T* b, O* out, uint64_t n, int sa, int sb) {
    constexpr uint64_t kChunk = (uint64_t)kEwThreads * VEC * kEwUnroll;
    const uint64_t base = (uint64_t)blockIdx.x * kChunk;
    if (base + kChunk <= n) {
        Vec<T, VEC> va[kEwUnroll], vb[kEwUnroll];
#pragma unroll
        for (int u = 0; u < kEwUnroll; u++) {
            uint64_t i = base + ((uint64_t)u * kEwThreads + threadIdx.x) * VEC;
            va[u] = sa ? ld_vec<T, VEC>(a + i) : splat<T, VEC>(a[0]);
            if constexpr (NIN == 2) vb[u] = sb ? ld_vec<T, VEC>(b + i) : splat<T, VEC>(b[0]);
        }
#pragma unroll
        for (int u = 0; u < kEwUnroll; u++) {
            uint64_t i = base + ((uint64_t)u * kEwThreads + threadIdx.x) * VEC;
            st_vec<O, VEC>(out + i, apply_vec<F, T, O, NIN, VEC>(f, va[u], vb[u]));
        }
    } else {
        for (uint64_t i = base + threadIdx.x; i < n; i += kEwThreads) {
            T x = a[sa ? i : 0];
            if constexpr (NIN == 2) out[i] = f(x, b[sb ? i : 0]);
            else out[i] = f(x);
        }
    }
}

// Funnel-shifts the 32 bytes (lo, hi) right by `sh` bytes and returns the low 16.
__device__ __forceinline__ uint4 shift_pair(const uint4& lo, const uint4& hi, uint32_t sh) {
    const uint32_t bits = (sh & 3u) * 8u;
    switch (sh >> 2) {
        case 0:
            return make_uint4(__funnelshift_r(lo.x, lo.y, bits), __funnelshift_r(lo.y, lo.z, bits), __funnelshift_r(lo.z, lo.w, bits),
                              __funnelshift_r(lo.w, hi.x, bits));
        case 1:
            return make_uint4(__funnelshift_r(lo.y, lo.z, bits), __funnelshift_r(lo.z, lo.w, bits), __funnelshift_r(lo.w, hi.x, bits),
                              __funnelshift_r(hi.x, hi.y, bits));
        case 2:
            return make_uint4(__funnelshift_r(lo.z, lo.w, bits), __funnelshift_r(lo.w, hi.x, bits), __funnelshift_r(hi.x, hi.y, bits),
                              __funnelshift_r(hi.y, hi.z, bits));
        default:
            return make_uint4(__funnelshift_r(lo.w, hi.x, bits), __funnelshift_r(hi.x, hi.y, bits), __funnelshift_r(hi.y, hi.z, bits),
                              __funnelshift_r(hi.z, hi.w, bits));
    }
}

// VEC elements starting at an arbitrary element-aligned address: the two aligned 16-byte words the vector straddles,
// shifted together.  `sh` = the address modulo 16 (the same for every vector of a launch).  Both words contain at
// least one byte of the vector, so neither load leaves the allocation.  The second word is the next lane's first
// word, so it comes from L1; handing it over by warp shuffle instead was measured slower (four shuffles per operand
// and vector cost more issue slots than the cached load).
template <class T, int VEC>
__device__ __forceinline__ Vec<T, VEC> ld_vec_shifted(const T* p, uint32_t sh) {
    static_assert(sizeof(T) * VEC == 16, "one 16-byte vector");
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p) - sh;
    const uint4 lo = *reinterpret_cast<const uint4*>(addr);
    if (sh == 0) return *reinterpret_cast<const Vec<T, VEC>*>(&lo);
    const uint4 hi = *reinterpret_cast<const uint4*>(addr + 16);
    const uint4 r = shift_pair(lo, hi, sh);
    return *reinterpret_cast<const Vec<T, VEC>*>(&r);
}

// Flat operands at addresses that are not 16-byte aligned.  Elements [0, head) and [tail_begin, n) are handled one at a
// time by block 0; the body [head, tail_begin) starts where the OUTPUT is aligned for its vector store, and each input
// is read with ld_vec_shifted (sha / shb = its address modulo 16 at the start of the body).  sa / sb: 1 = contiguous,
// 0 = broadcast scalar.
template <class F, class T, class O, int NIN, int VEC>
__global__ void __launch_bounds__(kEwThreads) ew_flat_shift_kernel(F f, const T* a, const T* b, O* out, uint64_t n, uint64_t head, uint64_t body_vecs,
                                                                   int sa, int sb, uint32_t sha, uint32_t shb) {
    const uint64_t v0 = (uint64_t)blockIdx.x * kEwThreads * kEwUnroll + threadIdx.x;
    Vec<T, VEC> va[kEwUnroll], vb[kEwUnroll];
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        const uint64_t v = v0 + (uint64_t)u * kEwThreads;
        if (v < body_vecs) {
            const uint64_t i = head + v * VEC;
            va[u] = sa ? ld_vec_shifted<T, VEC>(a + i, sha) : splat<T, VEC>(a[0]);
            if constexpr (NIN == 2) vb[u] = sb ? ld_vec_shifted<T, VEC>(b + i, shb) : splat<T, VEC>(b[0]);
        }
    }
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        const uint64_t v = v0 + (uint64_t)u * kEwThreads;
        if (v < body_vecs) st_vec<O, VEC>(out + head + v * VEC, apply_vec<F, T, O, NIN, VEC>(f, va[u], vb[u]));
    }
    if (blockIdx.x == 0) {
        const uint64_t tail_begin = head + body_vecs * VEC;
        const uint64_t edge = head + (n - tail_begin);  // fewer than VEC elements on either side
        for (uint64_t e = threadIdx.x; e < edge; e += kEwThreads) {
            const uint64_t i = e < head ? e : tail_begin + (e - head);
            T x = a[sa ? i : 0];
            if constexpr (NIN == 2) out[i] = f(x, b[sb ? i : 0]);
            else out[i] = f(x);
        }
    }
}

// The same work with the shifted operands staged through shared memory: one thread asks the copy engine of the SM
// (cp.async.bulk, global -> shared, completion on an mbarrier) for the 16-byte-aligned span that covers the block's part
// of each shifted operand - every byte crosses from L2 exactly once, in full lines - and each thread then assembles its
// vectors from two aligned 16-byte shared-memory words.  Used for large operands; the body of the block is kEwThreads *
// kEwUnroll vectors, i.e. 16 KB (+ 16 bytes) of shared memory per shifted operand.  The wait on the barrier is bounded.
constexpr int kEwStageBytes = kEwThreads * kEwUnroll * 16 + 16;

__device__ __forceinline__ bool ew_stage_wait(uint32_t bar, const tc::WaitReport& rep, int code) {
    for (int i = 0; i < (1 << 26); i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar)
            : "memory");
        if (ok) return true;
    }
    tc::wait_gave_up(rep, code);  // surfaces as status 5 at the caller's next synchronisation point
    return false;
}

template <class F, class T, class O, int NIN, int VEC>
__global__ void __launch_bounds__(kEwThreads) ew_flat_shift_staged_kernel(F f, const T* a, const T* b, O* out, uint64_t n, uint64_t head,
                                                                          uint64_t body_vecs, int sa, int sb, uint32_t sha, uint32_t shb, int stage_aligned, tc::WaitReport rep) {
    extern __shared__ __align__(128) unsigned char ew_stage[];
    __shared__ __align__(8) unsigned long long stage_bar;
    const uint64_t block_v0 = (uint64_t)blockIdx.x * kEwThreads * kEwUnroll;
    const uint64_t left = block_v0 < body_vecs ? body_vecs - block_v0 : 0;
    const uint32_t nv = left < (uint64_t)kEwThreads * kEwUnroll ? (uint32_t)left : (uint32_t)(kEwThreads * kEwUnroll);  // vectors of this block
    // stage_aligned: aligned operands go through shared memory as well (register-heavy functors keep too few loads in flight
    // on their own; the copy engine's queue does not depend on how many threads are resident)
    const bool stage_a = nv && sa && (sha != 0 || stage_aligned), stage_b = nv && NIN == 2 && sb && (shb != 0 || stage_aligned);
    unsigned char* buf_a = ew_stage;
    unsigned char* buf_b = ew_stage + (stage_a ? kEwStageBytes : 0);
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&stage_bar);
    if (stage_a || stage_b) {
        if (threadIdx.x == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // the aligned words the block's vectors straddle: one extra word only for an operand that is really shifted
            const uint32_t bytes_a = nv * 16 + (sha ? 16 : 0), bytes_b = nv * 16 + (shb ? 16 : 0);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((stage_a ? bytes_a : 0) + (stage_b ? bytes_b : 0)) : "memory");
            if (stage_a) {
                const uintptr_t src = reinterpret_cast<uintptr_t>(a + head + block_v0 * VEC) - sha;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 (uint32_t)__cvta_generic_to_shared(buf_a)),
                             "l"(src), "r"(bytes_a), "r"(bar)
                             : "memory");
            }
            if (stage_b) {
                const uintptr_t src = reinterpret_cast<uintptr_t>(b + head + block_v0 * VEC) - shb;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 (uint32_t)__cvta_generic_to_shared(buf_b)),
                             "l"(src), "r"(bytes_b), "r"(bar)
                             : "memory");
            }
        }
    }
    // operands that need no staging are read straight from global memory while the copies fly
    Vec<T, VEC> va[kEwUnroll], vb[kEwUnroll];
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        const uint32_t lv = (uint32_t)u * kEwThreads + threadIdx.x;
        if (lv < nv) {
            const uint64_t i = head + (block_v0 + lv) * VEC;
            if (!stage_a) va[u] = sa ? ld_vec<T, VEC>(a + i) : splat<T, VEC>(a[0]);
            if constexpr (NIN == 2)
                if (!stage_b) vb[u] = sb ? ld_vec<T, VEC>(b + i) : splat<T, VEC>(b[0]);
        }
    }
    bool landed = true;
    if (stage_a || stage_b) {
        __syncthreads();  // the barrier is initialised before anyone polls it
        landed = ew_stage_wait(bar, rep, 21);
    }
    if (landed) {
#pragma unroll
        for (int u = 0; u < kEwUnroll; u++) {
            const uint32_t lv = (uint32_t)u * kEwThreads + threadIdx.x;
            if (lv >= nv) continue;
            if (stage_a) {
                const uint4 lo = *reinterpret_cast<const uint4*>(buf_a + lv * 16);
                uint4 r = lo;
                if (sha) r = shift_pair(lo, *reinterpret_cast<const uint4*>(buf_a + lv * 16 + 16), sha);
                va[u] = *reinterpret_cast<const Vec<T, VEC>*>(&r);
            }
            if constexpr (NIN == 2) {
                if (stage_b) {
                    const uint4 lo = *reinterpret_cast<const uint4*>(buf_b + lv * 16);
                    uint4 r = lo;
                    if (shb) r = shift_pair(lo, *reinterpret_cast<const uint4*>(buf_b + lv * 16 + 16), shb);
                    vb[u] = *reinterpret_cast<const Vec<T, VEC>*>(&r);
                }
            }
            st_vec<O, VEC>(out + head + (block_v0 + lv) * VEC, apply_vec<F, T, O, NIN, VEC>(f, va[u], vb[u]));
        }
    }
    if (blockIdx.x == 0) {
        const uint64_t tail_begin = head + body_vecs * VEC;
        const uint64_t edge = head + (n - tail_begin);
        for (uint64_t e = threadIdx.x; e < edge; e += kEwThreads) {
            const uint64_t i = e < head ? e : tail_begin + (e - head);
            T x = a[sa ? i : 0];
            if constexpr (NIN == 2) out[i] = f(x, b[sb ? i : 0]);
            else out[i] = f(x);
        }
    }
}

struct EwRowParams {
    int nd_outer;
    uint32_t total_vecs;
    uint32_t qv;                    // vectors per row
    uint32_t chunks_per_row;        // long-row mode: blocks per row
    FastDiv qv_div;                 // short-row mode: vectors per row
    FastDiv chunk_div;              // long-row mode: blocks per row
    FastDiv outer_div[kMaxDims];    // outer dims, innermost outer dim last
    int64_t st[3][kMaxDims];        // outer strides per operand
    int sq[3];                      // stride along q per operand (1 or 0)
};

// Long rows (at least one block-load of vectors per row): a block works inside one row, so
// the row's base offsets are computed once per block and each thread only adds its vector
// index — the same instruction stream as the flat kernel.
template <class F, class T, class O, int NIN, int VEC>
__global__ void __launch_bounds__(kEwThreads, 4) ew_row_long_kernel(F f, const T* a, const T* b, O* out, EwRowParams P) {
    uint32_t r, chunk;
    P.chunk_div.divmod(blockIdx.x, r, chunk);
    int64_t o_out = 0, o_a = 0, o_b = 0;
    for (int d = P.nd_outer - 1; d >= 0; d--) {  // block-uniform
        uint32_t c;
        P.outer_div[d].divmod(r, r, c);
        o_out += (int64_t)c * P.st[0][d];
        o_a += (int64_t)c * P.st[1][d];
        if constexpr (NIN == 2) o_b += (int64_t)c * P.st[2][d];
    }
    out += o_out;
    a += o_a;
    if constexpr (NIN == 2) b += o_b;
    const uint32_t v0 = chunk * (kEwThreads * kEwUnroll) + threadIdx.x;
    Vec<T, VEC> va[kEwUnroll], vb[kEwUnroll];
    if (P.sq[1]) {
#pragma unroll
        for (int u = 0; u < kEwUnroll; u++)
            if (v0 + u * kEwThreads < P.qv) va[u] = ld_vec<T, VEC>(a + (size_t)(v0 + u * kEwThreads) * VEC);
    } else {
        Vec<T, VEC> s = splat<T, VEC>(a[0]);
#pragma unroll
        for (int u = 0; u < kEwUnroll; u++) va[u] = s;
    }
    if constexpr (NIN == 2) {
        if (P.sq[2]) {
#pragma unroll
            for (int u = 0; u < kEwUnroll; u++)
                if (v0 + u * kEwThreads < P.qv) vb[u] = ld_vec<T, VEC>(b + (size_t)(v0 + u * kEwThreads) * VEC);
        } else {
            Vec<T, VEC> s = splat<T, VEC>(b[0]);
#pragma unroll
            for (int u = 0; u < kEwUnroll; u++) vb[u] = s;
        }
    }
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        uint32_t v = v0 + u * kEwThreads;
        if (v < P.qv) st_vec<O, VEC>(out + (size_t)v * VEC, apply_vec<F, T, O, NIN, VEC>(f, va[u], vb[u]));
    }
}

// Unary op whose input is one row broadcast over every outer dim (strides [0, ..., 0, 1]):
// f(broadcast(x)) == broadcast(f(x)), so each thread evaluates its vectors once and stores
// them to a slab of output rows — the kernel is a pure store stream.
template <class F, class T, class O, int VEC>
__global__ void __launch_bounds__(kEwThreads) ew_bcast_rows_kernel(F f, const T* a, O* out, uint32_t qv, uint32_t rows, uint32_t rows_per_block) {
    const uint32_t v0 = blockIdx.x * (kEwThreads * kEwUnroll) + threadIdx.x;
    const uint32_t r0 = blockIdx.y * rows_per_block;
    const uint32_t r1 = min(rows, r0 + rows_per_block);
    Vec<O, VEC> res[kEwUnroll];
    Vec<T, VEC> dummy;
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        uint32_t v = v0 + u * kEwThreads;
        if (v < qv) res[u] = apply_vec<F, T, O, 1, VEC>(f, ld_vec<T, VEC>(a + (size_t)v * VEC), dummy);
    }
    for (uint32_t r = r0; r < r1; r++) {
        O* dst = out + (size_t)r * qv * VEC;
#pragma unroll
        for (int u = 0; u < kEwUnroll; u++) {
            uint32_t v = v0 + u * kEwThreads;
            if (v < qv) st_vec<O, VEC>(dst + (size_t)v * VEC, res[u]);
        }
    }
}

// The same store stream issued by the SM's copy engine: the block evaluates its chunk of the row into shared memory once
// and one thread then queues one cp.async.bulk (shared -> global) per output row of the block's slab; no per-element store
// instructions at all.  The chunk is kEwThreads * kEwUnroll output vectors (16 KB when the output type is as wide as the
// input type); rows are VEC * sizeof(O)-byte multiples here, so every copy is 16-byte aligned and sized.
template <class F, class T, class O, int VEC>
__global__ void __launch_bounds__(kEwThreads) ew_bcast_rows_bulk_kernel(F f, const T* a, O* out, uint32_t qv, uint32_t rows, uint32_t rows_per_block) {
    extern __shared__ __align__(128) unsigned char ew_stage[];
    const uint32_t chunk_v0 = blockIdx.x * (kEwThreads * kEwUnroll);
    const uint32_t nv = min(qv - chunk_v0, (uint32_t)(kEwThreads * kEwUnroll));
    const uint32_t r0 = blockIdx.y * rows_per_block;
    const uint32_t r1 = min(rows, r0 + rows_per_block);
    Vec<T, VEC> dummy;
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        const uint32_t lv = u * kEwThreads + threadIdx.x;
        if (lv < nv)
            *reinterpret_cast<Vec<O, VEC>*>(ew_stage + (size_t)lv * VEC * sizeof(O)) =
                apply_vec<F, T, O, 1, VEC>(f, ld_vec<T, VEC>(a + (size_t)(chunk_v0 + lv) * VEC), dummy);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copy engine reads what the threads just wrote
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t bytes = nv * VEC * (uint32_t)sizeof(O);
        const uint32_t src = (uint32_t)__cvta_generic_to_shared(ew_stage);
        for (uint32_t r = r0; r < r1; r++) {
            O* dst = out + ((size_t)r * qv + chunk_v0) * VEC;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // shared memory stays valid until the copies have read it (and landed)
    }
}

// Short rows: one fast-divmod per vector to find its row.
template <class F, class T, class O, int NIN, int VEC>
__global__ void __launch_bounds__(kEwThreads) ew_row_kernel(F f, const T* a, const T* b, O* out, EwRowParams P) {
    const uint32_t base = blockIdx.x * (kEwThreads * kEwUnroll);
#pragma unroll
    for (int u = 0; u < kEwUnroll; u++) {
        uint32_t v = base + u * kEwThreads + threadIdx.x;
        if (v < P.total_vecs) {
            uint32_t r, qv;
            P.qv_div.divmod(v, r, qv);
            int64_t o_out = (int64_t)qv * VEC, o_a = (int64_t)qv * VEC * P.sq[1], o_b = (int64_t)qv * VEC * P.sq[2];
#pragma unroll
            for (int d = kMaxDims - 1; d >= 0; d--) {
                if (d < P.nd_outer) {
                    uint32_t c;
                    P.outer_div[d].divmod(r, r, c);
                    o_out += (int64_t)c * P.st[0][d];
                    o_a += (int64_t)c * P.st[1][d];
                    if constexpr (NIN == 2) o_b += (int64_t)c * P.st[2][d];
                }
            }
            Vec<T, VEC> va = P.sq[1] ? ld_vec<T, VEC>(a + o_a) : splat<T, VEC>(a[o_a]), vb;
            if constexpr (NIN == 2) vb = P.sq[2] ? ld_vec<T, VEC>(b + o_b) : splat<T, VEC>(b[o_b]);
            st_vec<O, VEC>(out + o_out, apply_vec<F, T, O, NIN, VEC>(f, va, vb));
        }
    }
}

struct EwTileParams {
    uint32_t P, Q;                  // extents of the tiled dims
    uint32_t tiles_p, tiles_q;
    FastDiv tiles_q_div, tiles_p_div;
    int nd_batch;
    FastDiv batch_div[kMaxDims];
    int64_t st_batch[3][kMaxDims];
    int64_t st_p[3], st_q[3];
    int transposed[3];              // [1], [2]: input goes through shared memory
    int smem_slot[3];               // [1], [2]: which staging buffer a transposed input uses
};

template <class T>
struct EwTile {
    static constexpr int kTile = sizeof(T) == 8 ? 32 : 64;
    static constexpr int kPitch = kTile * (int)sizeof(T) + (sizeof(T) == 8 ? 8 : 4);  // bytes per staged row
    static constexpr int kBytes = kTile * kPitch;                                     // one staging buffer
};

// A warp covers 8 vectors x 4 rows (VEC > 1) or 32 elements x 1 row (VEC == 1) of the tile:
// 128-byte global segments, and shared-memory word accesses that do not collide.
template <int VPR, int VEC>
__device__ __forceinline__ void ew_tile_coord(int i, int& row, int& vcol) {
    if constexpr (VEC > 1 && VPR >= 8) {
        constexpr int WC = VPR / 8;  // warp-columns per tile row
        int w = i >> 5, lane = i & 31;
        vcol = (w % WC) * 8 + (lane & 7);
        row = (w / WC) * 4 + (lane >> 3);
    } else {
        row = i / VPR;
        vcol = i % VPR;
    }
}

template <class F, class T, class O, int NIN, int VEC>
__global__ void __launch_bounds__(kEwThreads, sizeof(T) == 2 ? 6 : 4) ew_tile_kernel(F f, const T* a, const T* b, O* out, EwTileParams P) {
    constexpr int TILE = EwTile<T>::kTile;
    constexpr int PITCH = EwTile<T>::kPitch;
    constexpr int VPR = TILE / VEC;                       // vectors per tile row
    constexpr int ITER = (TILE * VPR + kEwThreads - 1) / kEwThreads;
    extern __shared__ __align__(16) unsigned char ew_smem[];

    uint32_t t = blockIdx.x, tq, tp, bidx;
    P.tiles_q_div.divmod(t, t, tq);
    P.tiles_p_div.divmod(t, bidx, tp);
    int64_t base[3] = {0, 0, 0};
    for (int d = P.nd_batch - 1; d >= 0; d--) {  // block-uniform
        uint32_t c;
        P.batch_div[d].divmod(bidx, bidx, c);
#pragma unroll
        for (int k = 0; k < 3; k++) base[k] += (int64_t)c * P.st_batch[k][d];
    }
    const uint32_t p0 = tp * TILE, q0 = tq * TILE;
#pragma unroll
    for (int k = 0; k < 3; k++) base[k] += (int64_t)p0 * P.st_p[k] + (int64_t)q0 * P.st_q[k];
    const T* in[2] = {a, b};

    // Phase-2 work item: RP consecutive p-rows x one vector along q.  For 2-byte types two rows
    // are handled together, so that one 32-bit shared-memory read (two neighbouring p of one q)
    // feeds both: half the shared-memory instructions of a row-at-a-time walk.
    constexpr int RP = (sizeof(T) == 2 && VEC == 8) ? 2 : 1;
    constexpr int ITER2 = ((TILE / RP) * VPR + kEwThreads - 1) / kEwThreads;
    auto item_coord = [](int i, int& prow, int& qv) {
        if constexpr (RP == 2) {  // a warp covers 8 vectors (128 bytes) x 4 row pairs
            int w = i >> 5, lane = i & 31;
            qv = lane & 7;
            prow = (w * 4 + (lane >> 3)) * 2;
        } else {
            ew_tile_coord<VPR, VEC>(i, prow, qv);
        }
    };

    // All global loads of the tile are issued before the barrier: the direct operands in
    // the phase-2 mapping (rows along p, vectors along q), the transposed operands in the
    // phase-1 mapping (rows along q, vectors along p, their unit-stride dim).
    Vec<T, VEC> direct[NIN][ITER2][RP];
    Vec<T, VEC> staged[NIN][ITER];
#pragma unroll
    for (int x = 0; x < NIN; x++) {
        if (P.transposed[x + 1]) {
            const T* src = in[x] + base[x + 1];
#pragma unroll
            for (int it = 0; it < ITER; it++) {
                int qq, pv;
                ew_tile_coord<VPR, VEC>(threadIdx.x + it * kEwThreads, qq, pv);
                if (qq < TILE && q0 + qq < P.Q && p0 + pv * VEC < P.P) staged[x][it] = ld_vec<T, VEC>(src + (int64_t)qq * P.st_q[x + 1] + pv * VEC);
            }
        } else {
            const T* src = in[x] + base[x + 1];
#pragma unroll
            for (int it = 0; it < ITER2; it++) {
                int pp, qv;
                item_coord(threadIdx.x + it * kEwThreads, pp, qv);
#pragma unroll
                for (int r = 0; r < RP; r++) {
                    if (pp + r < TILE && p0 + pp + r < P.P && q0 + qv * VEC < P.Q) {
                        const T* s = src + (int64_t)(pp + r) * P.st_p[x + 1];
                        direct[x][it][r] = P.st_q[x + 1] ? ld_vec<T, VEC>(s + qv * VEC) : splat<T, VEC>(s[0]);
                    }
                }
            }
        }
    }
    // phase 1: stage the transposed inputs as [q][p]
#pragma unroll
    for (int x = 0; x < NIN; x++) {
        if (!P.transposed[x + 1]) continue;
        unsigned char* buf = ew_smem + P.smem_slot[x + 1] * EwTile<T>::kBytes;
#pragma unroll
        for (int it = 0; it < ITER; it++) {
            int qq, pv;
            ew_tile_coord<VPR, VEC>(threadIdx.x + it * kEwThreads, qq, pv);
            if (qq < TILE && q0 + qq < P.Q && p0 + pv * VEC < P.P) {
                unsigned char* row = buf + qq * PITCH + pv * VEC * (int)sizeof(T);
                if constexpr (VEC * sizeof(T) >= 4 && sizeof(T) < 4) {
                    const uint32_t* w = reinterpret_cast<const uint32_t*>(&staged[x][it]);
#pragma unroll
                    for (int j = 0; j < (int)(VEC * sizeof(T) / 4); j++) reinterpret_cast<uint32_t*>(row)[j] = w[j];
                } else {
#pragma unroll
                    for (int j = 0; j < VEC; j++) reinterpret_cast<T*>(row)[j] = staged[x][it].v[j];
                }
            }
        }
    }
    __syncthreads();

    // phase 2: walk the tile along q (the output's unit-stride dim)
#pragma unroll
    for (int it = 0; it < ITER2; it++) {
        int pp, qv;
        item_coord(threadIdx.x + it * kEwThreads, pp, qv);
        if (pp >= TILE || p0 + pp >= P.P || q0 + qv * VEC >= P.Q) continue;
        Vec<T, VEC> v[2][RP];
#pragma unroll
        for (int x = 0; x < NIN; x++) {
            if (P.transposed[x + 1]) {
                const unsigned char* buf = ew_smem + P.smem_slot[x + 1] * EwTile<T>::kBytes;
                if constexpr (RP == 2) {
                    // word j holds (q = qv*8 + j; p = pp, pp + 1): split the halves into the two rows
                    uint32_t w[VEC];
#pragma unroll
                    for (int j = 0; j < VEC; j++) w[j] = *reinterpret_cast<const uint32_t*>(buf + (qv * VEC + j) * PITCH + pp * 2);
                    uint32_t* r0 = reinterpret_cast<uint32_t*>(&v[x][0]);
                    uint32_t* r1 = reinterpret_cast<uint32_t*>(&v[x][1]);
#pragma unroll
                    for (int j = 0; j < VEC / 2; j++) {
                        r0[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x5410);
                        r1[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x7632);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < VEC; j++) v[x][0].v[j] = *reinterpret_cast<const T*>(buf + (qv * VEC + j) * PITCH + pp * (int)sizeof(T));
                }
            } else {
#pragma unroll
                for (int r = 0; r < RP; r++) v[x][r] = direct[x][it][r];
            }
        }
#pragma unroll
        for (int r = 0; r < RP; r++) {
            if (p0 + pp + r < P.P)
                st_vec<O, VEC>(out + base[0] + (int64_t)(pp + r) * P.st_p[0] + qv * VEC, apply_vec<F, T, O, NIN, VEC>(f, v[0][r], v[1][r]));
        }
    }
}

// Tile kernel for 2-byte element types (both in and out), vector-aligned layouts with at most one batch dim.  Every
// operand tile crosses between global and shared memory as ONE tensor copy (a 64 x 64 box, 128-byte swizzle; the inputs
// complete on an mbarrier, the output tile is written back the same way; ragged edges are clipped by the copy engine),
// so no thread spends load/store slots on global memory.  A transposed operand sits in shared memory as [q][p];
// ldmatrix.x4.trans hands each thread the 2 x 4 neighbouring-q pairs of one p-row, i.e. the transposition happens
// inside the instruction, and a direct operand and the output are read/written in that same fragment layout with
// 32-bit accesses.  Under the swizzle the eight 16-byte rows of an 8x8 block, and the 32 words of a fragment access,
// fall in distinct banks.
constexpr int kEwT16 = 64;
constexpr int kEwT16Bytes = kEwT16 * 128;

struct EwTile16Params {
    FastDiv tiles_q_div, tiles_p_div;
    int transposed[3];
    int batched[3];  // 0: the operand's map has one batch entry (broadcast along the batch dim)
};

template <class F, class T, class O, int NIN>
__global__ void __launch_bounds__(kEwThreads) ew_tile16_kernel(F f, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                               const __grid_constant__ CUtensorMap map_o, EwTile16Params P, tc::WaitReport rep) {
    static_assert(sizeof(T) == 2 && sizeof(O) == 2, "2-byte elements on both sides");
    extern __shared__ unsigned char ew_smem_raw[];
    __shared__ __align__(8) unsigned long long tile_bar;

    uint32_t t = blockIdx.x, tq, tp, bidx;
    P.tiles_q_div.divmod(t, t, tq);
    P.tiles_p_div.divmod(t, bidx, tp);
    const int p0 = (int)tp * kEwT16, q0 = (int)tq * kEwT16;
    const uint32_t smem0 = ((uint32_t)__cvta_generic_to_shared(ew_smem_raw) + 1023u) & ~1023u;  // the swizzle pattern repeats every 1024 bytes
    unsigned char* tiles = ew_smem_raw + (smem0 - (uint32_t)__cvta_generic_to_shared(ew_smem_raw));
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&tile_bar);

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)NIN * kEwT16Bytes) : "memory");
#pragma unroll
        for (int x = 0; x < NIN; x++) {
            const bool tr = P.transposed[x + 1] != 0;
            tc::tma_load_3d(smem0 + x * kEwT16Bytes, x ? &map_b : &map_a, tr ? p0 : q0, tr ? q0 : p0, P.batched[x + 1] ? (int)bidx : 0, bar);
        }
    }
    __syncthreads();  // the barrier is initialised before anyone polls it
    const bool landed = ew_stage_wait(bar, rep, 22);
    if (landed) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        unsigned char* obuf = tiles + NIN * kEwT16Bytes;
#pragma unroll
        for (int s = 0; s < 2; s++) {
            const int ws = warp + 8 * s, pb = ws >> 1, qh = ws & 1;  // an 8-row p-block x one 32-wide half of q per warp step
            // fragment word m of this lane: row p = pb*8 + lane/4, 16-byte chunk qh*4 + m (swizzled by the row), word lane%4
            const uint32_t frag_row = (uint32_t)(pb * 8 + (lane >> 2)) * 128u + (uint32_t)(lane & 3) * 4u;
            uint32_t w[2][4] = {};
#pragma unroll
            for (int x = 0; x < NIN; x++) {
                if (P.transposed[x + 1]) {
                    const uint32_t row = (uint32_t)(qh * 32 + lane);
                    const uint32_t addr = smem0 + x * kEwT16Bytes + row * 128u + (((uint32_t)pb ^ (row & 7u)) << 4);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w[x][0]), "=r"(w[x][1]), "=r"(w[x][2]), "=r"(w[x][3])
                                 : "r"(addr)
                                 : "memory");
                } else {
                    const unsigned char* src = tiles + x * kEwT16Bytes + frag_row;
#pragma unroll
                    for (int m = 0; m < 4; m++) w[x][m] = *reinterpret_cast<const uint32_t*>(src + (((uint32_t)(qh * 4 + m) ^ (uint32_t)(lane >> 2)) << 4));
                }
            }
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const Vec<O, 2> r = apply_vec<F, T, O, NIN, 2>(f, *reinterpret_cast<const Vec<T, 2>*>(&w[0][m]), *reinterpret_cast<const Vec<T, 2>*>(&w[1][m]));
                *reinterpret_cast<uint32_t*>(obuf + frag_row + (((uint32_t)(qh * 4 + m) ^ (uint32_t)(lane >> 2)) << 4)) = *reinterpret_cast<const uint32_t*>(&r);
            }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copy engine reads what the threads just wrote
    __syncthreads();
    if (landed && threadIdx.x == 0) {
        tc::tma_store_3d(&map_o, smem0 + NIN * kEwT16Bytes, q0, p0, (int)bidx);
        tc::tma_store_commit();
        tc::tma_store_wait_read<0>();  // shared memory stays valid until the copy has read it
    }
}

struct EwGenParams {
    int nd;
    uint64_t n;
    uint32_t dim[kMaxDims];
    FastDiv div[kMaxDims];
    int64_t st[3][kMaxDims];
};

template <class F, class T, class O, int NIN>
__global__ void __launch_bounds__(kEwThreads) ew_generic_kernel(F f, const T* a, const T* b, O* out, EwGenParams P) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < P.n; i += stride) {
        int64_t o0 = 0, o1 = 0, o2 = 0;
        if (P.n <= 0xFFFFFFFFull) {
            uint32_t r = (uint32_t)i;
            for (int d = P.nd - 1; d >= 0; d--) {
                uint32_t c;
                P.div[d].divmod(r, r, c);
                o0 += (int64_t)c * P.st[0][d];
                o1 += (int64_t)c * P.st[1][d];
                if constexpr (NIN == 2) o2 += (int64_t)c * P.st[2][d];
            }
        } else {
            uint64_t r = i;
            for (int d = P.nd - 1; d >= 0; d--) {
                uint64_t c = r % P.dim[d];
                r /= P.dim[d];
                o0 += (int64_t)c * P.st[0][d];
                o1 += (int64_t)c * P.st[1][d];
                if constexpr (NIN == 2) o2 += (int64_t)c * P.st[2][d];
            }
        }
        if constexpr (NIN == 2) out[o0] = f(a[o1], b[o2]);
        else out[o0] = f(a[o1]);
    }
}

// ---------------------------------------------------------------------------------
// launcher
// ---------------------------------------------------------------------------------
void ew_fill_row_params(const EwPlan& pl, int vec, EwRowParams& P);
void ew_fill_tile_params(const EwPlan& pl, int tile, EwTileParams& P, uint32_t& blocks);
void ew_fill_gen_params(const EwPlan& pl, EwGenParams& P);

// Host side of the 2-byte tile kernel: one tensor map per operand (rows along the operand's strided dim, columns along
// its unit-stride dim, the one batch dim as the third coordinate).  Returns false - nothing launched - for layouts the
// maps cannot express (a stride-0 or negative row pitch, two or more batch dims, a pitch the encoder rejects); the
// caller then runs the general tile kernel.
template <class F, class T, class O, int NIN>
bool ew_launch_tile16(const EwPlan& pl, const EwTileParams& TP, uint32_t blocks, const F& f, const T* a, const T* b, O* out, cudaStream_t s) {
    if (TP.nd_batch > 1) return false;
    const uint64_t nb = blocks / ((uint64_t)TP.tiles_p * TP.tiles_q);
    const void* base[3] = {out, a, b};
    CUtensorMap maps[3];
    EwTile16Params P;
    P.tiles_q_div = TP.tiles_q_div;
    P.tiles_p_div = TP.tiles_p_div;
    for (int k = 0; k <= NIN; k++) {
        const bool tr = k != 0 && TP.transposed[k];
        const uint64_t rows = tr ? TP.Q : TP.P, cols = tr ? TP.P : TP.Q;
        const int64_t pitch = tr ? TP.st_q[k] : TP.st_p[k], unit = tr ? TP.st_p[k] : TP.st_q[k];
        const int64_t bs = TP.nd_batch ? TP.st_batch[k][0] : 0;
        if (unit != 1 || pitch <= 0 || bs < 0 || (k == 0 && nb > 1 && bs == 0)) return false;
        P.transposed[k] = tr ? 1 : 0;
        P.batched[k] = (nb > 1 && bs != 0) ? 1 : 0;
        if (!tc::make_map_3d(&maps[k], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base[k], rows, cols, nb, (uint64_t)bs, kEwT16, CU_TENSOR_MAP_SWIZZLE_128B, (uint64_t)pitch))
            return false;
    }
    if (NIN == 1) {
        maps[2] = maps[1];
        P.transposed[2] = P.batched[2] = 0;
    }
    ew_tile16_kernel<F, T, O, NIN><<<blocks, kEwThreads, (NIN + 1) * kEwT16Bytes + 1024, s>>>(f, maps[1], maps[2], maps[0], P, tc::next_wait_report());
    return true;
}

template <class F, class T, class O, int NIN>
void ew_launch(const EwPlan& pl, const F& f, const T* a, const T* b, O* out, const char* where) {
    constexpr int VEC = 16 / sizeof(T);
    cudaStream_t s = ctx().stream;
    a += pl.off[1];
    if (NIN == 2) b += pl.off[2];
    out += pl.off[0];
    switch (pl.kind) {
        case EW_EMPTY:
            return;
        case EW_FLAT: {
            uint64_t chunk = (uint64_t)kEwThreads * VEC * kEwUnroll;
            uint64_t blocks = (pl.n + chunk - 1) / chunk;
            if (blocks > 0x7FFFFFFFull) {
                set_error(kErrUnsupported, 0, where);
                return;
            }
            if constexpr (F::kChecked) {
                // 16-bit division (approximate quotient + exact redo): 88 registers per thread leave few loads in flight, so
                // large operands are fed by bulk copies through shared memory instead
                const int sa = (int)pl.st[1][0], sb = NIN == 2 ? (int)pl.st[2][0] : 0;
                const int staged = (sa ? 1 : 0) + (sb ? 1 : 0);
                if (staged && pl.n / VEC >= 4096) {
                    ew_flat_shift_staged_kernel<F, T, O, NIN, VEC>
                        <<<(uint32_t)blocks, kEwThreads, (size_t)staged * kEwStageBytes, s>>>(f, a, b, out, pl.n, 0, pl.n / VEC, sa, sb, 0, 0, 1, tc::next_wait_report());
                    break;
                }
            }
            ew_flat_kernel<F, T, O, NIN, VEC><<<(uint32_t)blocks, kEwThreads, 0, s>>>(f, a, b, out, pl.n, (int)pl.st[1][0], NIN == 2 ? (int)pl.st[2][0] : 0);
            break;
        }
        case EW_FLAT_SHIFT: {
            // head: elements until the output reaches the alignment of its vector store
            const uintptr_t oaddr = reinterpret_cast<uintptr_t>(out);
            const size_t oalign = VEC * sizeof(O);
            uint64_t head = ((oalign - oaddr % oalign) % oalign) / sizeof(O);
            if (head > pl.n) head = pl.n;
            const uint64_t body_vecs = (pl.n - head) / VEC;
            const int sa = (int)pl.st[1][0], sb = NIN == 2 ? (int)pl.st[2][0] : 0;
            const uint32_t sha = sa ? (uint32_t)(reinterpret_cast<uintptr_t>(a + head) % 16) : 0;
            const uint32_t shb = (NIN == 2 && sb) ? (uint32_t)(reinterpret_cast<uintptr_t>(b + head) % 16) : 0;
            uint64_t blocks = (body_vecs + (uint64_t)kEwThreads * kEwUnroll - 1) / ((uint64_t)kEwThreads * kEwUnroll);
            if (blocks == 0) blocks = 1;
            if (blocks > 0x7FFFFFFFull) {
                set_error(kErrUnsupported, 0, where);
                return;
            }
            const int staged = (sa && sha != 0 ? 1 : 0) + (NIN == 2 && sb && shb != 0 ? 1 : 0);
            if (staged && body_vecs >= 4096) {
                // large operands: the shifted ones go through shared memory, one bulk copy per block and operand
                ew_flat_shift_staged_kernel<F, T, O, NIN, VEC>
                    <<<(uint32_t)blocks, kEwThreads, (size_t)staged * kEwStageBytes, s>>>(f, a, b, out, pl.n, head, body_vecs, sa, sb, sha, shb, 0, tc::next_wait_report());
                break;
            }
            ew_flat_shift_kernel<F, T, O, NIN, VEC><<<(uint32_t)blocks, kEwThreads, 0, s>>>(f, a, b, out, pl.n, head, body_vecs, sa, sb, sha, shb);
            break;
        }
        case EW_ROW: {
            EwRowParams P;
            ew_fill_row_params(pl, VEC, P);
            uint64_t rows = P.total_vecs / P.qv;
            bool row_bcast = NIN == 1 && P.nd_outer == 1 && P.sq[1] == 1 && P.st[1][0] == 0 && P.st[0][0] == (int64_t)P.qv * VEC && rows >= 8;
            if constexpr (NIN == 1) {
                if (row_bcast) {
                    // enough blocks to fill the GPU, each storing a slab of rows
                    uint32_t want = (uint32_t)sm_count() * 8;
                    uint32_t gy = (want + P.chunks_per_row - 1) / P.chunks_per_row;
                    if (gy > rows) gy = (uint32_t)rows;
                    if (gy > 65535) gy = 65535;
                    uint32_t rpb = (uint32_t)((rows + gy - 1) / gy);
                    gy = (uint32_t)((rows + rpb - 1) / rpb);
                    if ((VEC * sizeof(O)) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
                        const size_t stage = (size_t)kEwThreads * kEwUnroll * VEC * sizeof(O);
                        ew_bcast_rows_bulk_kernel<F, T, O, VEC><<<dim3(P.chunks_per_row, gy), kEwThreads, stage, s>>>(f, a, out, P.qv, (uint32_t)rows, rpb);
                        break;
                    }
                    ew_bcast_rows_kernel<F, T, O, VEC><<<dim3(P.chunks_per_row, gy), kEwThreads, 0, s>>>(f, a, out, P.qv, (uint32_t)rows, rpb);
                    break;
                }
            }
            if (P.qv >= (uint32_t)kEwThreads && rows * P.chunks_per_row < 0x7FFFFFFFull) {
                ew_row_long_kernel<F, T, O, NIN, VEC><<<(uint32_t)(rows * P.chunks_per_row), kEwThreads, 0, s>>>(f, a, b, out, P);
            } else {
                uint32_t blocks = ceil_div_u32(P.total_vecs, kEwThreads * kEwUnroll);
                ew_row_kernel<F, T, O, NIN, VEC><<<blocks, kEwThreads, 0, s>>>(f, a, b, out, P);
            }
            break;
        }
        case EW_TILE: {
            EwTileParams P;
            uint32_t blocks;
            ew_fill_tile_params(pl, EwTile<T>::kTile, P, blocks);
            int nslots = (P.transposed[1] ? 1 : 0) + (P.transposed[2] ? 1 : 0);
            size_t smem = (size_t)nslots * EwTile<T>::kBytes;
            if constexpr (sizeof(T) == 2 && sizeof(O) == 2) {
                if (pl.vec && ew_launch_tile16<F, T, O, NIN>(pl, P, blocks, f, a, b, out, s)) break;
            }
            if (pl.vec) ew_tile_kernel<F, T, O, NIN, VEC><<<blocks, kEwThreads, smem, s>>>(f, a, b, out, P);
            else ew_tile_kernel<F, T, O, NIN, 1><<<blocks, kEwThreads, smem, s>>>(f, a, b, out, P);
            break;
        }
        case EW_GENERIC:
        case EW_SERIAL: {
            EwGenParams P;
            ew_fill_gen_params(pl, P);
            if (pl.kind == EW_SERIAL) {
                ew_generic_kernel<F, T, O, NIN><<<1, 1, 0, s>>>(f, a, b, out, P);
            } else {
                uint64_t blocks = (pl.n + kEwThreads - 1) / kEwThreads;
                uint64_t cap = (uint64_t)sm_count() * 32;
                if (blocks > cap) blocks = cap;
                ew_generic_kernel<F, T, O, NIN><<<(uint32_t)blocks, kEwThreads, 0, s>>>(f, a, b, out, P);
            }
            break;
        }
        default:
            set_error(kErrBadMetadata, 0, where);
            return;
    }
    check_launch(where);
}

// Entry points used by the C-ABI wrappers.  `meta` is the pointer the caller passed
// (device or host memory, or NULL for "contiguous, no offsets").
template <class Op, class T, class O>
void binary_entry(size_t n, size_t nd, const size_t* meta, const T* lhs, const T* rhs, O* out, bool inplace, const char* where) {
    const size_t* hm = meta ? resolve_metadata(meta, 3 * nd + 2) : nullptr;
    if (meta && !hm) return;
    EwPlan pl;
    ew_make_plan(pl, n, nd, hm, 2, inplace, sizeof(T), sizeof(O), out, lhs, rhs);
    ew_launch<Binary<Op, T, O>, T, O, 2>(pl, Binary<Op, T, O>(), lhs, rhs, out, where);
}
template <class Op, class T, class O>
void unary_entry(size_t n, size_t nd, const size_t* meta, const T* in, O* out, const char* where) {
    const size_t* hm = meta ? resolve_metadata(meta, 2 * nd + 1) : nullptr;
    if (meta && !hm) return;
    // The reference accepts input == NULL as "read from the output buffer"; that is
    // only meaningful when input and output have the same element type.
    if (!in) in = reinterpret_cast<const T*>(out);
    EwPlan pl;
    ew_make_plan(pl, n, nd, hm, 1, false, sizeof(T), sizeof(O), out, in, nullptr);
    ew_launch<Unary<Op, T, O>, T, O, 1>(pl, Unary<Op, T, O>(), in, (const T*)nullptr, out, where);
}
template <class Op, class T, class O>
void unary_const_entry(size_t n, size_t nd, const size_t* meta, const T* in, T c, O* out, const char* where) {
    const size_t* hm = meta ? resolve_metadata(meta, 2 * nd + 1) : nullptr;
    if (meta && !hm) return;
    if (!in) in = reinterpret_cast<const T*>(out);
    EwPlan pl;
    ew_make_plan(pl, n, nd, hm, 1, false, sizeof(T), sizeof(O), out, in, nullptr);
    UnaryConst<Op, T, O> f;
    f.c = c;
    ew_launch<UnaryConst<Op, T, O>, T, O, 1>(pl, f, in, (const T*)nullptr, out, where);
}

}  // namespace mx
