// The remaining families of the reference's CUDA crate: fold (the backward of unfold), the three
// paddings with their backward passes, and softmax.  Each has a general kernel that follows the
// reference's index formulas for any layout (one thread per output element for fold and the
// paddings, one block per slice for softmax) and, for the common layouts, a faster form: softmax
// rows held in registers and a column form, paddings with a compile-time rank and 16-byte output
// vectors, the constant padding's backward as a cropped copy.  All keep the contracts of the rest
// of the library: outputs are overwritten (no pre-zero assumption), accumulation is wide (f32 for
// 16-bit floats, wrapping for integers) with one final rounding, and loops that the reference
// leaves unbounded are bounded here.
//   fold      crates/maidenx_cpu/src/ops/reduction.rs:274-381   kernels/ops/reduction.cu:169-241
//   padding   crates/maidenx_cpu/src/ops/padding.rs             kernels/ops/padding.cu
//   softmax   crates/maidenx_cpu/src/nn/activation/softmax.rs   kernels/nn/activation/softmax.cu
#include "abi_common.cuh"
#include "ops.cuh"
#include "reduction.cuh"

namespace mx {

constexpr int kExThreads = 256;
constexpr int kExMaxDims = 8;

static unsigned ex_blocks(u64 n) {
    u64 b = (n + kExThreads - 1) / kExThreads;
    u64 cap = (u64)sm_count() * 32;
    if (b > cap) b = cap;
    return b ? (unsigned)b : 1u;
}

// ---------------------------------------------------------------------------------
// fold: out[..., w * step + p, ...] += in[..., w, ..., p, ...], written as a gather so that the
// result is deterministic: every output element adds its windows in ascending window order.
// ---------------------------------------------------------------------------------
struct FoldParams {
    int nd;
    u64 dims[kExMaxDims], strides[kExMaxDims];
    int fold_dim, window_dim;
    u64 fold_size, step, num_els, off, out_size;
};

template <class T>
__global__ void __launch_bounds__(kExThreads) fold_kernel(const T* in, T* out, FoldParams P) {
    typedef typename SumAcc<T>::type Acc;
    const u64 stride = (u64)gridDim.x * kExThreads;
    for (u64 j = (u64)blockIdx.x * kExThreads + threadIdx.x; j < P.out_size; j += stride) {
        // output coordinates: the input dims without the window dim, fold_dim of extent fold_size
        u64 coord[kExMaxDims];
        u64 r = j;
        for (int d = P.nd - 1; d >= 0; d--) {
            if (d == P.window_dim) continue;
            const u64 ext = d == P.fold_dim ? P.fold_size : P.dims[d];
            coord[d] = r % ext;
            r /= ext;
        }
        const u64 pos = coord[P.fold_dim];
        u64 base = 0;
        for (int d = 0; d < P.nd; d++)
            if (d != P.window_dim && d != P.fold_dim) base += coord[d] * P.strides[d];
        Acc acc = (Acc)0;
        const u64 nwin = P.dims[P.fold_dim], wsize = P.dims[P.window_dim];
        // windows w with 0 <= pos - w * step < window size
        u64 w_lo = pos >= wsize ? (pos - wsize + P.step) / P.step : 0;
        for (u64 w = w_lo; w < nwin && w * P.step <= pos; w++) {
            const u64 p = pos - w * P.step;
            if (p >= wsize) continue;
            u64 src = (base + w * P.strides[P.fold_dim] + p * P.strides[P.window_dim]) % P.num_els;  // the reference wraps the source index
            acc = acc + RedTraits<T, RED_SUM>::load(in[P.off + src]);
        }
        out[j] = RedTraits<T, RED_SUM>::finalize(acc, 1);
    }
}

// The same gather with 32-bit arithmetic for inputs below 2^32 elements whose largest source index stays inside the
// buffer (every dense layout and every view unfold() makes): multiply-shift divisions, no wrap of the source index.
struct FoldFastParams {
    int nd, fold_dim, window_dim;
    FastDiv out_div[kExMaxDims];  // by the output extents (fold_dim: fold_size; window_dim unused)
    u32 strides[kExMaxDims];
    u32 nwin, wsize, step, out_size;
    u64 off;
};

template <class T>
__global__ void __launch_bounds__(kExThreads) fold_fast_kernel(const T* __restrict__ in, T* __restrict__ out, FoldFastParams P) {
    typedef typename SumAcc<T>::type Acc;
    const u32 j = blockIdx.x * kExThreads + threadIdx.x;
    if (j >= P.out_size) return;
    u32 r = j, pos = 0, base = 0;
    for (int d = P.nd - 1; d >= 0; d--) {
        if (d == P.window_dim) continue;
        u32 c;
        P.out_div[d].divmod(r, r, c);
        if (d == P.fold_dim) pos = c;
        else base += c * P.strides[d];
    }
    const T* src = in + P.off + base;
    Acc acc = (Acc)0;
    // windows w with 0 <= pos - w * step < window size, in ascending order
    const u32 w_lo = pos >= P.wsize ? (pos - P.wsize + P.step) / P.step : 0;
    for (u32 w = w_lo; w < P.nwin && w * P.step <= pos; w++) {
        const u32 p = pos - w * P.step;
        if (p >= P.wsize) continue;
        acc = acc + RedTraits<T, RED_SUM>::load(src[w * P.strides[P.fold_dim] + p * P.strides[P.window_dim]]);
    }
    out[j] = RedTraits<T, RED_SUM>::finalize(acc, 1);
}

template <class T>
void fold_entry(size_t num_els, size_t nd, const size_t* meta, const T* in, T* out, const char* where) {
    const size_t* hm = resolve_metadata(meta, 2 * nd + 6);
    if (!hm || nd == 0 || nd > (size_t)kExMaxDims) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    FoldParams P;
    P.nd = (int)nd;
    for (size_t d = 0; d < nd; d++) {
        P.dims[d] = hm[d];
        P.strides[d] = hm[nd + d];
    }
    P.fold_dim = (int)hm[2 * nd];
    P.window_dim = (int)hm[2 * nd + 1];
    P.fold_size = hm[2 * nd + 2];
    P.step = hm[2 * nd + 3];
    P.off = hm[2 * nd + 5];
    P.num_els = num_els;
    if (P.fold_dim < 0 || P.fold_dim >= P.nd || P.window_dim < 0 || P.window_dim >= P.nd || P.fold_dim == P.window_dim || P.step == 0 || num_els == 0) {
        if (num_els == 0) return;
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    P.out_size = 1;
    for (int d = 0; d < P.nd; d++) {
        if (d == P.window_dim) continue;
        P.out_size *= d == P.fold_dim ? P.fold_size : P.dims[d];
    }
    if (P.out_size == 0) return;
    {
        // largest source index of the layout; the reference wraps indices at num_els, which a layout inside the buffer never needs
        u64 max_src = 0;
        bool fits = num_els < (1ull << 32) && P.out_size < (1ull << 32) && P.fold_size < (1ull << 31) && P.step < (1ull << 31);
        for (int d = 0; d < P.nd && fits; d++) {
            fits = P.dims[d] > 0 && P.dims[d] < (1ull << 31) && P.strides[d] < (1ull << 32);
            if (fits) max_src += (P.dims[d] - 1) * P.strides[d];
        }
        if (fits && max_src < num_els) {
            FoldFastParams F;
            F.nd = P.nd;
            F.fold_dim = P.fold_dim;
            F.window_dim = P.window_dim;
            for (int d = 0; d < P.nd; d++) {
                F.out_div[d].init((u32)(d == P.fold_dim ? P.fold_size : P.dims[d]));
                F.strides[d] = (u32)P.strides[d];
            }
            F.nwin = (u32)P.dims[P.fold_dim];
            F.wsize = (u32)P.dims[P.window_dim];
            F.step = (u32)P.step;
            F.out_size = (u32)P.out_size;
            F.off = P.off;
            fold_fast_kernel<T><<<(unsigned)((P.out_size + kExThreads - 1) / kExThreads), kExThreads, 0, ctx().stream>>>(in, out, F);
            check_launch(where);
            return;
        }
    }
    fold_kernel<T><<<ex_blocks(P.out_size), kExThreads, 0, ctx().stream>>>(in, out, P);
    check_launch(where);
}

// ---------------------------------------------------------------------------------
// padding
// metadata: [in_dims(n) | in_strides(n) | in_offset | out_dims(n) | (before, after) x n]
// ---------------------------------------------------------------------------------
enum { PAD_CONSTANT = 0, PAD_REFLECTION = 1, PAD_REPLICATION = 2 };

struct PadParams {
    int nd;
    int contiguous;
    u64 in_dims[kExMaxDims], in_strides[kExMaxDims], out_dims[kExMaxDims], before[kExMaxDims];
    u64 in_off, n_in, n_out;
};

// Input coordinate of output coordinate oc along one dim; false = outside (constant padding).
template <int MODE>
__device__ __forceinline__ bool pad_source(long long oc, long long before, long long size, u64& ic) {
    long long pos = oc - before;
    if (MODE == PAD_CONSTANT) {
        if (pos < 0 || pos >= size) return false;
    } else if (MODE == PAD_REFLECTION) {
        // the reference loops until the position is inside; pads >= the dim size are rejected above this
        // layer, and a size-1 dim would never terminate, so the walk is bounded
        for (int guard = 0; (pos < 0 || pos >= size) && guard < 64; guard++) pos = pos < 0 ? -pos : 2 * size - pos - 2;
        if (pos < 0 || pos >= size) pos = 0;
    } else {
        pos = pos < 0 ? 0 : (pos > size - 1 ? size - 1 : pos);
    }
    ic = (u64)pos;
    return true;
}

template <int MODE>
__device__ __forceinline__ bool pad_in_index(u64 i, const PadParams& P, u64& idx) {
    u64 oc[kExMaxDims];
    u64 r = i;
    for (int d = P.nd - 1; d >= 0; d--) {
        oc[d] = r % P.out_dims[d];
        r /= P.out_dims[d];
    }
    u64 lin = 0, str = 0, mul = 1;
    bool inside = true;
    for (int d = P.nd - 1; d >= 0; d--) {
        u64 ic;
        if (!pad_source<MODE>((long long)oc[d], (long long)P.before[d], (long long)P.in_dims[d], ic)) {
            inside = false;
            break;
        }
        lin += ic * mul;
        mul *= P.in_dims[d];
        str += ic * P.in_strides[d];
    }
    idx = P.contiguous ? lin : str;
    return inside;
}

template <class T, int MODE>
__global__ void __launch_bounds__(kExThreads) pad_forward_kernel(const T* in, T* out, T pad_value, PadParams P) {
    const u64 stride = (u64)gridDim.x * kExThreads;
    for (u64 i = (u64)blockIdx.x * kExThreads + threadIdx.x; i < P.n_out; i += stride) {
        u64 idx;
        out[i] = pad_in_index<MODE>(i, P, idx) ? in[P.in_off + idx] : pad_value;
    }
}

// Backward: every grad_out element is added to the input position it was read from.  Wide atomics into
// a zeroed workspace, then one pass that rounds and overwrites grad_in[in_off .. in_off + n_in).
template <class T, int MODE>
__global__ void __launch_bounds__(kExThreads) pad_backward_scatter_kernel(const T* grad_out, typename SumAcc<T>::type* ws, PadParams P) {
    const u64 stride = (u64)gridDim.x * kExThreads;
    for (u64 i = (u64)blockIdx.x * kExThreads + threadIdx.x; i < P.n_out; i += stride) {
        u64 idx;
        if (pad_in_index<MODE>(i, P, idx) && idx < P.n_in) atomic_combine_sum(ws + idx, RedTraits<T, RED_SUM>::load(grad_out[i]));
    }
}

// The same gather for the common sizes (outputs below 2^32 elements, at most four dims after size-1 dims are dropped and
// neighbouring unpadded dims merged - an [N, C, H, W] batch padded along H and W is [N*C, H, W]): the rank is a
// compile-time constant, so coordinates live in registers, all index arithmetic is 32-bit, and a thread produces one
// 16-byte vector of consecutive output elements: the output index is split once per vector (multiply-shift division),
// the outer dims' source offset is kept while the last coordinate advances and recomputed only when it wraps.
constexpr int kPadFastDims = 4;
struct PadFastParams {
    int nd;
    FastDiv div[kPadFastDims];                                              // forward: by out_dims; crop: by in_dims
    u32 out_dims[kPadFastDims], in_dims[kPadFastDims], before[kPadFastDims];
    u64 mul[kPadFastDims];                                                  // forward: element step per input dim; crop: per grad_out dim
    u64 in_off;
    u32 n_out, n_in;
};

template <int MODE>
__device__ __forceinline__ bool pad_source32(int oc, int before, int size, int& ic) {
    int pos = oc - before;
    if (MODE == PAD_CONSTANT) {
        if (pos < 0 || pos >= size) return false;
    } else if (MODE == PAD_REFLECTION) {
        // one fold is enough for pads below the dim size (the only ones the layers above let through); the bounded
        // walk of the general kernel covers the rest
        if (pos < 0) pos = -pos;
        else if (pos >= size) pos = 2 * size - pos - 2;
        if (pos < 0 || pos >= size) {
            for (int guard = 0; (pos < 0 || pos >= size) && guard < 64; guard++) pos = pos < 0 ? -pos : 2 * size - pos - 2;
            if (pos < 0 || pos >= size) pos = 0;
        }
    } else {
        pos = pos < 0 ? 0 : (pos > size - 1 ? size - 1 : pos);
    }
    ic = pos;
    return true;
}

template <class T, int MODE, int ND>
__global__ void __launch_bounds__(kExThreads) pad_forward_fast_kernel(const T* __restrict__ in, T* __restrict__ out, T pad_value, PadFastParams P) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int last = ND - 1;
    const u64 v0 = ((u64)blockIdx.x * kExThreads + threadIdx.x) * VEC;
    if (v0 >= P.n_out) return;
    u32 oc[ND];
    u32 r = (u32)v0;
#pragma unroll
    for (int d = last; d >= 0; d--) P.div[d].divmod(r, r, oc[d]);
    bool outer_in = true;
    u64 outer_base = P.in_off;
    auto outer = [&]() {
        outer_in = true;
        outer_base = P.in_off;
#pragma unroll
        for (int d = 0; d < last; d++) {
            int ic = 0;
            outer_in = outer_in && pad_source32<MODE>((int)oc[d], (int)P.before[d], (int)P.in_dims[d], ic);
            outer_base += (u64)(u32)ic * P.mul[d];
        }
    };
    outer();
    Vec<T, VEC> res;
    const u32 count = P.n_out - (u32)v0 < (u32)VEC ? P.n_out - (u32)v0 : (u32)VEC;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        if ((u32)j < count) {
            int ic = 0;
            const bool inside = pad_source32<MODE>((int)oc[last], (int)P.before[last], (int)P.in_dims[last], ic) && outer_in;
            res.v[j] = inside ? in[outer_base + (u64)(u32)ic * P.mul[last]] : pad_value;
            if (++oc[last] == P.out_dims[last]) {
                oc[last] = 0;
                bool carry = true;
#pragma unroll
                for (int d = last - 1; d >= 0; d--) {
                    if (carry) {
                        if (++oc[d] < P.out_dims[d]) carry = false;
                        else oc[d] = 0;
                    }
                }
                outer();
            }
        }
    }
    if (count == (u32)VEC && reinterpret_cast<uintptr_t>(out + v0) % 16 == 0) {
        *reinterpret_cast<Vec<T, VEC>*>(out + v0) = res;
    } else {
#pragma unroll
        for (int j = 0; j < VEC; j++)
            if ((u32)j < count) out[v0 + j] = res.v[j];
    }
}

// Image batches ([planes, H, W] after merging, padded along H and W only, contiguous planes).  The map from a position
// of the output plane to its source position in the input plane (-1: the fill value) is the same for every plane, so a
// small kernel writes it once into the scratch block; the main kernel (1- and 2-byte types: after staging a few whole
// input planes in shared memory with flat 16-byte loads) writes its output planes in order, each lane 32 bits' worth of
// neighbouring elements (one f32, two 16-bit, four 8-bit values - one store where the address allows): per element one
// table read, one read of the source and a select - no coordinate arithmetic in the inner loop.
struct PadPlaneParams {
    u32 planes, H, W, Ho, Wo, before_h, before_w;
    u32 planes_per_block;
    u32 src_plane, dst_plane;  // elements per input / output plane
    u64 src_off, dst_off;      // element offsets of the first plane in the two buffers
};

template <int MODE>
__global__ void __launch_bounds__(kExThreads) pad_plane_table_kernel(int* __restrict__ table, PadPlaneParams P) {
    const u32 e = blockIdx.x * kExThreads + threadIdx.x;
    if (e >= P.Ho * P.Wo) return;
    const u32 oh = e / P.Wo, ow = e - oh * P.Wo;
    int ih = 0, iw = 0;
    const bool inside = pad_source32<MODE>((int)oh, (int)P.before_h, (int)P.H, ih) && pad_source32<MODE>((int)ow, (int)P.before_w, (int)P.W, iw);
    table[e] = inside ? ih * (int)P.W + iw : -1;
}

template <class T>
__global__ void __launch_bounds__(kExThreads) pad_planes_kernel(const T* __restrict__ in, T* __restrict__ out, T pad_value, const int* __restrict__ table, PadPlaneParams P) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int EPL = sizeof(T) >= 4 ? 1 : 4 / (int)sizeof(T);
    extern __shared__ __align__(16) unsigned char pad_smem[];
    T* tile = reinterpret_cast<T*>(pad_smem);
    const u32 p0 = blockIdx.x * P.planes_per_block;
    const u32 np = P.planes - p0 < P.planes_per_block ? P.planes - p0 : P.planes_per_block;
    const u32 in_plane = P.src_plane, out_plane = P.dst_plane;
    const T* src = in + P.src_off + (u64)p0 * in_plane;
    T* dst = out + P.dst_off + (u64)p0 * out_plane;
    const u32 n_in = np * in_plane;
    // 1- and 2-byte elements are staged (their gathers would be 2-byte global loads: measured 2.7 TB/s against 4.1
    // staged); wider elements are read in place (5.0 TB/s against 4.4 staged: the near-contiguous gather coalesces)
    constexpr bool STAGED = sizeof(T) < 4;
    if (!STAGED) {
    } else if (reinterpret_cast<uintptr_t>(src) % 16 == 0) {
        const u32 nv = n_in / VEC;
        for (u32 v = threadIdx.x; v < nv; v += kExThreads) reinterpret_cast<Vec<T, VEC>*>(tile)[v] = reinterpret_cast<const Vec<T, VEC>*>(src)[v];
        for (u32 e = nv * VEC + threadIdx.x; e < n_in; e += kExThreads) tile[e] = src[e];
    } else {
        for (u32 e = threadIdx.x; e < n_in; e += kExThreads) tile[e] = src[e];
    }
    if (STAGED) __syncthreads();
    for (u32 pl = 0; pl < np; pl++) {
        const T* splane = (STAGED ? tile : src) + (u64)pl * in_plane;
        T* oplane = dst + (u64)pl * out_plane;
        if (EPL > 1 && reinterpret_cast<uintptr_t>(oplane) % 4 == 0) {
            const u32 body = out_plane / EPL * EPL;
            for (u32 r = threadIdx.x * EPL; r < body; r += kExThreads * EPL) {
                Vec<T, EPL> v;
#pragma unroll
                for (int j = 0; j < EPL; j++) {
                    const int idx = __ldg(table + r + j);
                    v.v[j] = idx >= 0 ? splane[idx] : pad_value;
                }
                *reinterpret_cast<uint32_t*>(oplane + r) = *reinterpret_cast<const uint32_t*>(&v);
            }
            for (u32 r = body + threadIdx.x; r < out_plane; r += kExThreads) {
                const int idx = __ldg(table + r);
                oplane[r] = idx >= 0 ? splane[idx] : pad_value;
            }
        } else {
            for (u32 r = threadIdx.x; r < out_plane; r += kExThreads) {
                const int idx = __ldg(table + r);
                oplane[r] = idx >= 0 ? splane[idx] : pad_value;
            }
        }
    }
}

// Backward of constant padding over a contiguous input: every input element was read by exactly one output element,
// so the gradient is a cropped copy - no accumulation, no workspace.
template <class T, int ND>
__global__ void __launch_bounds__(kExThreads) pad_constant_backward_crop_kernel(const T* __restrict__ grad_out, T* __restrict__ grad_in, PadFastParams P) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int last = ND - 1;
    const u64 v0 = ((u64)blockIdx.x * kExThreads + threadIdx.x) * VEC;
    if (v0 >= P.n_in) return;
    u32 ic[ND];
    u32 r = (u32)v0;
#pragma unroll
    for (int d = last; d >= 0; d--) P.div[d].divmod(r, r, ic[d]);
    auto outer = [&]() {
        u64 base = 0;
#pragma unroll
        for (int d = 0; d < last; d++) base += (u64)(ic[d] + P.before[d]) * P.mul[d];
        return base;
    };
    u64 outer_base = outer();
    Vec<T, VEC> res;
    const u32 count = P.n_in - (u32)v0 < (u32)VEC ? P.n_in - (u32)v0 : (u32)VEC;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        if ((u32)j < count) {
            res.v[j] = grad_out[outer_base + (u64)(ic[last] + P.before[last]) * P.mul[last]];
            if (++ic[last] == P.in_dims[last]) {
                ic[last] = 0;
                bool carry = true;
#pragma unroll
                for (int d = last - 1; d >= 0; d--) {
                    if (carry) {
                        if (++ic[d] < P.in_dims[d]) carry = false;
                        else ic[d] = 0;
                    }
                }
                outer_base = outer();
            }
        }
    }
    T* dst = grad_in + P.in_off + v0;
    if (count == (u32)VEC && reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
        *reinterpret_cast<Vec<T, VEC>*>(dst) = res;
    } else {
#pragma unroll
        for (int j = 0; j < VEC; j++)
            if ((u32)j < count) dst[j] = res.v[j];
    }
}

// Fills F from P for the forward gather (crop = false: `mul` = input steps, `div` by out_dims) or the cropped copy
// (crop = true: `mul` = dense grad_out steps, `div` by in_dims).  Returns false when the shape does not fit the fast form.
static bool pad_fast_params(PadFastParams& F, const PadParams& P, bool crop);

static bool pad_params(PadParams& P, size_t n_in, size_t n_out, size_t nd, const size_t* meta, const char* where) {
    const size_t* hm = resolve_metadata(meta, 5 * nd + 1);
    if (!hm || nd > (size_t)kExMaxDims) {
        set_error(kErrBadMetadata, 0, where);
        return false;
    }
    P.nd = (int)nd;
    for (size_t d = 0; d < nd; d++) {
        P.in_dims[d] = hm[d];
        P.in_strides[d] = hm[nd + d];
        P.out_dims[d] = hm[2 * nd + 1 + d];
        P.before[d] = hm[3 * nd + 1 + 2 * d];
        if (P.out_dims[d] == 0 || P.in_dims[d] == 0) return false;  // nothing to do
    }
    P.in_off = hm[2 * nd];
    P.n_in = n_in;
    P.n_out = n_out;
    // crates/maidenx_cpu/src/utils.rs:2-12: size-1 dims are ignored
    size_t acc = 1;
    P.contiguous = 1;
    for (size_t d = nd; d-- > 0;) {
        if (P.in_dims[d] > 1 && P.in_strides[d] != acc) P.contiguous = 0;
        acc *= P.in_dims[d];
    }
    return true;
}

static bool pad_fast_params(PadFastParams& F, const PadParams& P, bool crop) {
    if (P.nd < 1 || P.n_out >= (1ull << 32) || P.n_in >= (1ull << 32)) return false;
    if (crop && !P.contiguous) return false;
    u64 in_step[kExMaxDims], out_step[kExMaxDims], in_total = 1, out_total = 1;
    for (int d = P.nd - 1; d >= 0; d--) {
        if (P.out_dims[d] >= (1ull << 31) || P.in_dims[d] >= (1ull << 31) || P.before[d] >= (1ull << 31)) return false;
        if (crop && P.before[d] + P.in_dims[d] > P.out_dims[d]) return false;  // a source outside grad_out
        in_step[d] = P.contiguous ? in_total : P.in_strides[d];
        out_step[d] = out_total;
        in_total *= P.in_dims[d];
        out_total *= P.out_dims[d];
    }
    if (out_total != P.n_out || (crop && in_total != P.n_in)) return false;
    int k = 0;
    bool prev_plain = false;
    for (int d = 0; d < P.nd; d++) {
        if (P.in_dims[d] == 1 && P.out_dims[d] == 1) continue;  // contributes nothing to either index
        const bool plain = P.in_dims[d] == P.out_dims[d] && P.before[d] == 0;
        // an unpadded dim joins the unpadded dim before it when the two are one run in the source
        if (plain && prev_plain && F.mul[k - 1] == (crop ? out_step[d] * P.out_dims[d] : in_step[d] * P.in_dims[d]) && (u64)F.in_dims[k - 1] * P.in_dims[d] < (1ull << 31)) {
            F.in_dims[k - 1] *= (u32)P.in_dims[d];
            F.out_dims[k - 1] = F.in_dims[k - 1];
            F.mul[k - 1] = crop ? out_step[d] : in_step[d];
        } else {
            if (k == kPadFastDims) return false;
            F.in_dims[k] = (u32)P.in_dims[d];
            F.out_dims[k] = (u32)P.out_dims[d];
            F.before[k] = (u32)P.before[d];
            F.mul[k] = crop ? out_step[d] : in_step[d];
            k++;
        }
        prev_plain = plain;
    }
    if (k == 0) {  // every dim has extent 1
        F.in_dims[0] = F.out_dims[0] = 1;
        F.before[0] = 0;
        F.mul[0] = 1;
        k = 1;
    }
    F.nd = k;
    for (int d = 0; d < k; d++) F.div[d].init(crop ? F.in_dims[d] : F.out_dims[d]);
    F.in_off = P.in_off;
    F.n_out = (u32)P.n_out;
    F.n_in = (u32)P.n_in;
    return true;
}

template <class T, int MODE>
void pad_forward_entry(size_t n_in, size_t n_out, size_t nd, const size_t* meta, const T* in, T* out, T pad_value, const char* where) {
    if (n_out == 0) return;
    PadParams P;
    if (!pad_params(P, n_in, n_out, nd, meta, where)) return;
    PadFastParams F;
    if (pad_fast_params(F, P, false)) {
        constexpr int VEC = 16 / (int)sizeof(T);
        // [planes, H, W] with unpadded, contiguous planes of at most 24 KB: staged through shared memory
        if (F.nd == 3 && F.in_dims[0] == F.out_dims[0] && F.before[0] == 0 && F.mul[2] == 1 && F.mul[1] == F.in_dims[2] &&
            F.mul[0] == (u64)F.in_dims[1] * F.in_dims[2] && (u64)F.in_dims[1] * F.in_dims[2] * sizeof(T) <= 24 * 1024 && F.in_dims[0] >= 64) {
            PadPlaneParams Q;
            Q.planes = F.in_dims[0];
            Q.H = F.in_dims[1];
            Q.W = F.in_dims[2];
            Q.Ho = F.out_dims[1];
            Q.Wo = F.out_dims[2];
            Q.before_h = F.before[1];
            Q.before_w = F.before[2];
            const u32 plane_bytes = Q.H * Q.W * (u32)sizeof(T);
            Q.planes_per_block = 24 * 1024 / plane_bytes;
            // a whole 16-byte multiple of input per block keeps every block's staging loads on the vector form
            while (Q.planes_per_block > 1 && (Q.planes_per_block * plane_bytes) % 16 != 0) Q.planes_per_block--;
            Q.src_plane = Q.H * Q.W;
            Q.dst_plane = Q.Ho * Q.Wo;
            Q.src_off = F.in_off;
            Q.dst_off = 0;
            int* table = (u64)Q.Ho * Q.Wo < (1ull << 24) ? static_cast<int*>(scratch((size_t)Q.Ho * Q.Wo * sizeof(int))) : nullptr;
            if (table) {
                const unsigned blocks = (Q.planes + Q.planes_per_block - 1) / Q.planes_per_block;
                cudaStream_t st = ctx().stream;
                pad_plane_table_kernel<MODE><<<(Q.Ho * Q.Wo + kExThreads - 1) / kExThreads, kExThreads, 0, st>>>(table, Q);
                pad_planes_kernel<T><<<blocks, kExThreads, sizeof(T) < 4 ? Q.planes_per_block * plane_bytes : 0, st>>>(in, out, pad_value, table, Q);
                check_launch(where);
                return;
            }
        }
        const unsigned blocks = (unsigned)(((n_out + VEC - 1) / VEC + kExThreads - 1) / kExThreads);
        cudaStream_t st = ctx().stream;
        switch (F.nd) {
            case 1: pad_forward_fast_kernel<T, MODE, 1><<<blocks, kExThreads, 0, st>>>(in, out, pad_value, F); break;
            case 2: pad_forward_fast_kernel<T, MODE, 2><<<blocks, kExThreads, 0, st>>>(in, out, pad_value, F); break;
            case 3: pad_forward_fast_kernel<T, MODE, 3><<<blocks, kExThreads, 0, st>>>(in, out, pad_value, F); break;
            default: pad_forward_fast_kernel<T, MODE, 4><<<blocks, kExThreads, 0, st>>>(in, out, pad_value, F); break;
        }
        check_launch(where);
        return;
    }
    pad_forward_kernel<T, MODE><<<ex_blocks(n_out), kExThreads, 0, ctx().stream>>>(in, out, pad_value, P);
    check_launch(where);
}

template <class T, int MODE>
void pad_backward_entry(size_t n_in, size_t n_out, size_t nd, const size_t* meta, const T* grad_out, T* grad_in, const char* where) {
    typedef typename SumAcc<T>::type Acc;
    if (n_in == 0) return;
    PadParams P;
    if (!pad_params(P, n_in, n_out, nd, meta, where)) return;
    PadFastParams F;
    if (MODE == PAD_CONSTANT && pad_fast_params(F, P, true)) {
        constexpr int VEC = 16 / (int)sizeof(T);
        const unsigned blocks = (unsigned)(((n_in + VEC - 1) / VEC + kExThreads - 1) / kExThreads);
        cudaStream_t st = ctx().stream;
        switch (F.nd) {
            case 1: pad_constant_backward_crop_kernel<T, 1><<<blocks, kExThreads, 0, st>>>(grad_out, grad_in, F); break;
            case 2: pad_constant_backward_crop_kernel<T, 2><<<blocks, kExThreads, 0, st>>>(grad_out, grad_in, F); break;
            case 3: pad_constant_backward_crop_kernel<T, 3><<<blocks, kExThreads, 0, st>>>(grad_out, grad_in, F); break;
            default: pad_constant_backward_crop_kernel<T, 4><<<blocks, kExThreads, 0, st>>>(grad_out, grad_in, F); break;
        }
        check_launch(where);
        return;
    }
    Acc* ws = static_cast<Acc*>(scratch(sizeof(Acc) * n_in));
    if (!ws) return;
    cudaStream_t s = ctx().stream;
    reduce_fill_kernel<T, RED_SUM><<<ex_blocks(n_in), kRedThreads, 0, s>>>(ws, n_in);
    if (n_out) pad_backward_scatter_kernel<T, MODE><<<ex_blocks(n_out), kExThreads, 0, s>>>(grad_out, ws, P);
    reduce_finalize_kernel<T, RED_SUM><<<ex_blocks(n_in), kRedThreads, 0, s>>>(ws, grad_in + P.in_off, n_in, 1);
    check_launch(where);
}

// ---------------------------------------------------------------------------------
// softmax along one dim: out[pre, i, post] = exp(x - max) / sum(exp(x - max)); one block per
// (pre, post) slice, three passes over the slice (max, sum, quotient), f32 arithmetic for 16-bit
// inputs and f64 for f64.  The output is contiguous; the input is indexed as the reference does.
// ---------------------------------------------------------------------------------
struct SoftmaxParams {
    int nd, dim, contiguous;
    u64 dims[kExMaxDims], strides[kExMaxDims];
    u64 off, pre, n, post;
};

__device__ __forceinline__ u64 softmax_index(const SoftmaxParams& P, u64 pre_idx, u64 i, u64 post_idx) {
    if (P.contiguous) return P.off + pre_idx * (P.n * P.post) + i * P.post + post_idx;
    u64 idx = P.off, rem = pre_idx;
    for (int d = 0; d < P.dim; d++) {  // the reference peels the leading dims in ascending order (softmax.rs:123-128)
        idx += (rem % P.dims[d]) * P.strides[d];
        rem /= P.dims[d];
    }
    idx += i * P.strides[P.dim];
    rem = post_idx;
    for (int d = P.nd - 1; d > P.dim; d--) {
        idx += (rem % P.dims[d]) * P.strides[d];
        rem /= P.dims[d];
    }
    return idx;
}

template <class T>
__global__ void __launch_bounds__(kExThreads) softmax_kernel(const T* in, T* out, SoftmaxParams P) {
    typedef typename std::conditional<std::is_same<T, f64>::value, f64, f32>::type A;
    typedef RedTraits<A, RED_MAX> MaxT;
    typedef RedTraits<A, RED_SUM> SumT;
    __shared__ A s_bcast;
    for (u64 slice = blockIdx.x; slice < P.pre * P.post; slice += gridDim.x) {
        const u64 pre_idx = slice / P.post, post_idx = slice - pre_idx * P.post;
        auto value = [&](u64 i) -> A {
            const T v = in[softmax_index(P, pre_idx, i, post_idx)];
            if constexpr (is_half_v<T>) return to_f32(v);
            else return (A)v;
        };
        A mx = -INFINITY;
        for (u64 i = threadIdx.x; i < P.n; i += kExThreads) {
            const A v = value(i);
            mx = v > mx ? v : mx;  // the reference's comparison: a NaN never becomes the maximum
        }
        mx = block_reduce<MaxT, kExThreads>(mx);
        if (threadIdx.x == 0) s_bcast = mx;
        __syncthreads();
        mx = s_bcast;
        __syncthreads();
        A sum = (A)0;
        for (u64 i = threadIdx.x; i < P.n; i += kExThreads) {
            if constexpr (std::is_same<A, f64>::value) sum += exp(value(i) - mx);
            else sum += expf(value(i) - mx);
        }
        sum = block_reduce<SumT, kExThreads>(sum);
        if (threadIdx.x == 0) s_bcast = sum;
        __syncthreads();
        sum = s_bcast;
        __syncthreads();
        for (u64 i = threadIdx.x; i < P.n; i += kExThreads) {
            A e;
            if constexpr (std::is_same<A, f64>::value) e = exp(value(i) - mx);
            else e = expf(value(i) - mx);
            const A q = e / sum;
            T r;
            if constexpr (is_half_v<T>) r = from_f32<T>(q);
            else r = (T)q;
            out[pre_idx * (P.n * P.post) + i * P.post + post_idx] = r;
        }
    }
}

// Contiguous input, softmax along the last dim, rows short enough for the registers of their thread group (a warp for
// rows up to 8 vectors per lane, else the block): every element is read once and written once, as 16-byte vectors.
// Same formulas as above (comparison-based maximum, exp(x - max), quotient by the sum); the sum is a tree over the
// group instead of the block-strided partial sums.
__device__ __forceinline__ float exp2_approx(float v) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v));
    return e;
}

template <class A, int G, bool IS_MAX>
__device__ __forceinline__ A softmax_group_all(A v, A* part) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const A w = __shfl_xor_sync(0xFFFFFFFFu, v, o);
        v = IS_MAX ? (w > v ? w : v) : v + w;
    }
    if constexpr (G > 32) {  // `part` is used once per kernel (the maximum and the sum have one each)
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
        __syncthreads();
        v = part[0];
#pragma unroll
        for (int w = 1; w < G / 32; w++) v = IS_MAX ? (part[w] > v ? part[w] : v) : v + part[w];
    }
    return v;
}

template <class T, int G, int K>
__global__ void __launch_bounds__(kExThreads, (K * 16 / (int)sizeof(T) <= 32) ? 5 : 1) softmax_rows_kernel(const T* __restrict__ in, T* __restrict__ out, u64 rows, u32 n) {
    typedef typename std::conditional<std::is_same<T, f64>::value, f64, f32>::type A;
    constexpr int VEC = 16 / (int)sizeof(T);
    __shared__ A part_max[kExThreads / 32], part_sum[kExThreads / 32];
    const int t = threadIdx.x % G;
    const u64 row = (u64)blockIdx.x * (kExThreads / G) + threadIdx.x / G;
    if (G == 32 && row >= rows) return;  // whole warps; the warp form uses no block barrier
    const T* src = in + row * n;
    A x[K][VEC];
    A mx = -INFINITY;
    Vec<T, VEC> raw[K];
#pragma unroll
    for (int k = 0; k < K; k++) {  // every load of the row is issued before the first value is used
        const u32 i = (u32)(k * G + t) * VEC;
        if (i < n) raw[k] = *reinterpret_cast<const Vec<T, VEC>*>(src + i);
    }
#pragma unroll
    for (int k = 0; k < K; k++) {
        if ((u32)(k * G + t) * VEC < n) {
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                if constexpr (is_half_v<T>) x[k][j] = to_f32(raw[k].v[j]);
                else x[k][j] = (A)raw[k].v[j];
                mx = x[k][j] > mx ? x[k][j] : mx;  // a NaN never becomes the maximum
            }
        }
    }
    mx = softmax_group_all<A, G, true>(mx, part_max);
    A sum = (A)0;
#pragma unroll
    for (int k = 0; k < K; k++) {
        if ((u32)(k * G + t) * VEC < n) {
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                if constexpr (std::is_same<A, f64>::value) x[k][j] = exp(x[k][j] - mx);
                // f32 and 16-bit: the hardware exp2 of (x - max) * log2(e).  The product's rounding error is |t| * 2^-24 in the
                // exponent: at most 5e-6 relative for the smallest results an f32 can hold (t = -126), below 1e-6 down to
                // exp(-20) - inside the f32 tolerance everywhere, far below a 16-bit step
                else x[k][j] = exp2_approx((x[k][j] - mx) * 1.4426950408889634f);
                sum += x[k][j];
            }
        }
    }
    sum = softmax_group_all<A, G, false>(sum, part_sum);
    // f32 / 16-bit: one reciprocal per row and a multiply per element (within 1.5 ulp of the quotient); f64 divides
    const A inv = (A)1 / sum;
    T* dst = out + row * n;
#pragma unroll
    for (int k = 0; k < K; k++) {
        const u32 i = (u32)(k * G + t) * VEC;
        if (i < n) {
            Vec<T, VEC> r;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                A q;
                if constexpr (std::is_same<A, f64>::value) q = x[k][j] / sum;
                else q = x[k][j] * inv;
                if constexpr (is_half_v<T>) r.v[j] = from_f32<T>(q);
                else r.v[j] = (T)q;
            }
            *reinterpret_cast<Vec<T, VEC>*>(dst + i) = r;
        }
    }
}

// Contiguous input, softmax along a dim that is not the last: a block covers LANES x VEC neighbouring (pre, post)
// columns - 128 bytes of every row it touches: 8 lanes of 16-byte vectors when the extent of the trailing dims allows,
// else 32 lanes of single elements - with 256 / LANES threads per column group, which take every (256 / LANES)-th
// element of the dim, four loads in flight each, and combine through shared memory; three passes as in the general kernel.
template <class T, int VEC, int LANES>
__global__ void __launch_bounds__(kExThreads) softmax_cols_kernel(const T* __restrict__ in, T* __restrict__ out, u64 pre, u64 n, u64 post) {
    typedef typename std::conditional<std::is_same<T, f64>::value, f64, f32>::type A;
    constexpr int kSmColLanes = LANES, kSmColRows = kExThreads / LANES;
    __shared__ A part[kSmColRows][kSmColLanes][VEC];
    const int lane = threadIdx.x % kSmColLanes, ry = threadIdx.x / kSmColLanes;
    const u64 col = ((u64)blockIdx.x * kSmColLanes + lane) * VEC;  // VEC divides post: a vector stays inside one pre index
    const bool live = col < pre * post;
    const u64 pre_idx = live ? col / post : 0, post_idx = live ? col - pre_idx * post : 0;
    const T* src = in + pre_idx * n * post + post_idx;
    T* dst = out + pre_idx * n * post + post_idx;
    auto load = [&](u64 i, A (&v)[VEC]) {
        const Vec<T, VEC> raw = *reinterpret_cast<const Vec<T, VEC>*>(src + i * post);
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            if constexpr (is_half_v<T>) v[j] = to_f32(raw.v[j]);
            else v[j] = (A)raw.v[j];
        }
    };
    auto exp_of = [](A v) -> A {
        if constexpr (std::is_same<A, f64>::value) return exp(v);
        else return expf(v);
    };
    auto column_all = [&](A (&v)[VEC], bool is_max) {
        __syncthreads();  // the previous use of `part` has been read
#pragma unroll
        for (int j = 0; j < VEC; j++) part[ry][lane][j] = v[j];
        __syncthreads();
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            A r = part[0][lane][j];
#pragma unroll
            for (int k = 1; k < kSmColRows; k++) r = is_max ? (part[k][lane][j] > r ? part[k][lane][j] : r) : r + part[k][lane][j];
            v[j] = r;
        }
    };
    A mx[VEC], sum[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        mx[j] = -INFINITY;
        sum[j] = (A)0;
    }
    if (live) {
#pragma unroll 4
        for (u64 i = ry; i < n; i += kSmColRows) {
            A v[VEC];
            load(i, v);
#pragma unroll
            for (int j = 0; j < VEC; j++) mx[j] = v[j] > mx[j] ? v[j] : mx[j];
        }
    }
    column_all(mx, true);
    if (live) {
#pragma unroll 4
        for (u64 i = ry; i < n; i += kSmColRows) {
            A v[VEC];
            load(i, v);
#pragma unroll
            for (int j = 0; j < VEC; j++) sum[j] += exp_of(v[j] - mx[j]);
        }
    }
    column_all(sum, false);
    if (live) {
#pragma unroll 4
        for (u64 i = ry; i < n; i += kSmColRows) {
            A v[VEC];
            load(i, v);
            Vec<T, VEC> r;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                const A q = exp_of(v[j] - mx[j]) / sum[j];
                if constexpr (is_half_v<T>) r.v[j] = from_f32<T>(q);
                else r.v[j] = (T)q;
            }
            *reinterpret_cast<Vec<T, VEC>*>(dst + i * post) = r;
        }
    }
}

template <class T, int G>
bool softmax_rows_launch(const T* in, T* out, u64 rows, u32 n, cudaStream_t s) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int KMAX = sizeof(T) == 2 ? 8 : 16;  // at most 64 values per thread
    const u32 vecs = (n / VEC + G - 1) / G;          // vectors per thread
    const unsigned blocks = (unsigned)((rows + kExThreads / G - 1) / (kExThreads / G));
    if (vecs <= 1) softmax_rows_kernel<T, G, 1><<<blocks, kExThreads, 0, s>>>(in, out, rows, n);
    else if (vecs <= 2) softmax_rows_kernel<T, G, 2><<<blocks, kExThreads, 0, s>>>(in, out, rows, n);
    else if (vecs <= 4) softmax_rows_kernel<T, G, 4><<<blocks, kExThreads, 0, s>>>(in, out, rows, n);
    else if (vecs <= 8) softmax_rows_kernel<T, G, 8><<<blocks, kExThreads, 0, s>>>(in, out, rows, n);
    else if (KMAX >= 16 && vecs <= 16) softmax_rows_kernel<T, G, (KMAX >= 16 ? 16 : 8)><<<blocks, kExThreads, 0, s>>>(in, out, rows, n);
    else return false;
    return true;
}

template <class T>
void softmax_entry(size_t num_els, size_t nd, size_t dim, const size_t* meta, const T* in, T* out, const char* where) {
    if (!meta || !in || !out || nd == 0 || num_els == 0) return;  // the reference returns silently
    const size_t* hm = resolve_metadata(meta, 2 * nd + 1);
    if (!hm || nd > (size_t)kExMaxDims) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    SoftmaxParams P;
    P.nd = (int)nd;
    P.dim = (int)(dim >= nd ? nd - 1 : dim);
    P.pre = P.post = 1;
    for (size_t d = 0; d < nd; d++) {
        P.dims[d] = hm[d];
        P.strides[d] = hm[nd + d];
        if ((int)d < P.dim) P.pre *= hm[d];
        if ((int)d > P.dim) P.post *= hm[d];
    }
    P.n = hm[P.dim];
    P.off = hm[2 * nd];
    P.contiguous = 1;  // softmax.rs:86-98: this test does not skip size-1 dims
    size_t acc = 1;
    for (size_t d = nd; d-- > 0;) {
        if (P.strides[d] != acc) {
            P.contiguous = 0;
            break;
        }
        acc *= P.dims[d];
    }
    const u64 slices = P.pre * P.post;
    if (slices == 0 || P.n == 0) return;
    cudaStream_t st = ctx().stream;
    if (P.contiguous && slices < (1ull << 31) * 8) {
        constexpr int VEC = 16 / (int)sizeof(T);
        const T* src = in + P.off;
        const bool vec_ok = P.n % VEC == 0 && P.n < (1ull << 31) && (reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
        if (P.post == 1 && vec_ok && P.pre < (1ull << 31)) {
            const bool done = P.n <= 32ull * VEC * 8 ? softmax_rows_launch<T, 32>(src, out, P.pre, (u32)P.n, st)
                                                     : softmax_rows_launch<T, kExThreads>(src, out, P.pre, (u32)P.n, st);
            if (done) {
                check_launch(where);
                return;
            }
        }
        if (P.post >= 16) {
            const bool wide = P.post % VEC == 0 && (reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
            if (wide) softmax_cols_kernel<T, VEC, 8><<<(unsigned)((slices / VEC + 7) / 8), kExThreads, 0, st>>>(src, out, P.pre, P.n, P.post);
            else softmax_cols_kernel<T, 1, 32><<<(unsigned)((slices + 31) / 32), kExThreads, 0, st>>>(src, out, P.pre, P.n, P.post);
            check_launch(where);
            return;
        }
    }
    u64 blocks = slices < (u64)sm_count() * 16 ? slices : (u64)sm_count() * 16;
    softmax_kernel<T><<<(unsigned)blocks, kExThreads, 0, ctx().stream>>>(in, out, P);
    check_launch(where);
}

}  // namespace mx

using namespace mx;

#ifndef MX_T
#error "compile with -DMX_T=<dtype suffix> -DMX_TCLASS=<class>"
#endif

#define MX_EX_ARITH_(T)                                                                                                                          \
    void cuda_fold_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o) { fold_entry<mx_##T>(n, nd, m, i, o, "cuda_fold_" #T); } \
    void cuda_pad_with_constant_##T(size_t ni, size_t no, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o, mx_##T##_arg c) {              \
        pad_forward_entry<mx_##T, PAD_CONSTANT>(ni, no, nd, m, i, o, scalar_arg<mx_##T>(c), "cuda_pad_with_constant_" #T);                        \
    }                                                                                                                                            \
    void cuda_pad_with_reflection_##T(size_t ni, size_t no, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o) {                             \
        pad_forward_entry<mx_##T, PAD_REFLECTION>(ni, no, nd, m, i, o, scalar_arg<mx_##T>((mx_##T##_arg)0), "cuda_pad_with_reflection_" #T);      \
    }                                                                                                                                            \
    void cuda_pad_with_replication_##T(size_t ni, size_t no, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o) {                            \
        pad_forward_entry<mx_##T, PAD_REPLICATION>(ni, no, nd, m, i, o, scalar_arg<mx_##T>((mx_##T##_arg)0), "cuda_pad_with_replication_" #T);    \
    }                                                                                                                                            \
    void cuda_pad_with_constant_backward_##T(size_t ni, size_t no, size_t nd, const size_t* m, const mx_##T* g, mx_##T* gi) {                     \
        pad_backward_entry<mx_##T, PAD_CONSTANT>(ni, no, nd, m, g, gi, "cuda_pad_with_constant_backward_" #T);                                   \
    }                                                                                                                                            \
    void cuda_pad_with_reflection_backward_##T(size_t ni, size_t no, size_t nd, const size_t* m, const mx_##T* g, mx_##T* gi) {                   \
        pad_backward_entry<mx_##T, PAD_REFLECTION>(ni, no, nd, m, g, gi, "cuda_pad_with_reflection_backward_" #T);                               \
    }                                                                                                                                            \
    void cuda_pad_with_replication_backward_##T(size_t ni, size_t no, size_t nd, const size_t* m, const mx_##T* g, mx_##T* gi) {                  \
        pad_backward_entry<mx_##T, PAD_REPLICATION>(ni, no, nd, m, g, gi, "cuda_pad_with_replication_backward_" #T);                             \
    }
#define MX_EX_ARITH(T) MX_EX_ARITH_(T)
#define MX_EX_FLOAT_(T)                                                                                              \
    void cuda_softmax_##T(size_t n, size_t nd, size_t dim, const size_t* m, const mx_##T* i, mx_##T* o) {            \
        softmax_entry<mx_##T>(n, nd, dim, m, i, o, "cuda_softmax_" #T);                                              \
    }
#define MX_EX_FLOAT(T) MX_EX_FLOAT_(T)

extern "C" {
MX_EX_ARITH(MX_T)
#if MX_TCLASS == MX_CLASS_FLOAT
MX_EX_FLOAT(MX_T)
#endif
}
