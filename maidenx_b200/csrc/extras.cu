// The remaining families of the reference's CUDA crate: fold (the backward of unfold), the three
// paddings with their backward passes, and softmax.  They are not on the benchmarked path; the
// kernels are plain and correct rather than tuned - one thread per output element for fold and
// the paddings, one block per slice for softmax - and they keep the contracts of
// the rest of the library: outputs are overwritten (no pre-zero assumption), accumulation is
// wide (f32 for 16-bit floats, wrapping for integers) with one final rounding, and loops that
// the reference leaves unbounded are bounded here.
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

template <class T, int MODE>
void pad_forward_entry(size_t n_in, size_t n_out, size_t nd, const size_t* meta, const T* in, T* out, T pad_value, const char* where) {
    if (n_out == 0) return;
    PadParams P;
    if (!pad_params(P, n_in, n_out, nd, meta, where)) return;
    pad_forward_kernel<T, MODE><<<ex_blocks(n_out), kExThreads, 0, ctx().stream>>>(in, out, pad_value, P);
    check_launch(where);
}

template <class T, int MODE>
void pad_backward_entry(size_t n_in, size_t n_out, size_t nd, const size_t* meta, const T* grad_out, T* grad_in, const char* where) {
    typedef typename SumAcc<T>::type Acc;
    if (n_in == 0) return;
    PadParams P;
    if (!pad_params(P, n_in, n_out, nd, meta, where)) return;
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
