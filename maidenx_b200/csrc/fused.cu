// Fused elementwise passes of the MLP training step (additive mx_* exports, no counterpart in
// the reference's crate).  Each replaces a chain of single-op calls the reference's autograd
// issues, with the same formulas:
//   mx_bias_gelu       u = z + b ; a = gelu(u)          Linear's bias add (crates/maidenx_nn/src/layers/linear.rs:76-78)
//                                                        + GELU forward (crates/maidenx_cpu/src/ops/unary.rs:268-293)
//   mx_bias_add        u = z + b                         last layer (no activation)
//   mx_gelu_backward   du = dy * gelu'(u)                the 15-op closure at crates/maidenx_tensor/src/ops/unary.rs:324-346
//   mx_mse_loss_grad   loss = mean((p - t)^2), dp = 2 (p - t) / n   crates/maidenx_nn/src/losses/mse.rs:21-29 and its backward
//   mx_sgd_update      w32 -= lr * scale * g ; w16 = round(w32)      crates/maidenx_nn/src/optimizers/sgd.rs:17-26 with an
//                                                        f32 master copy of the 16-bit weights
// All are HBM-bound: 16-byte vector accesses, four vectors in flight per thread, math in f32,
// one rounding per stored value.
#include "abi_common.cuh"
#include "ops.cuh"
#include "matmul_tc.cuh"

namespace mx {

constexpr int kFusedThreads = 256;

template <class T>
__device__ __forceinline__ float ld_scalar_f32(const T* p) {
    if constexpr (is_half_v<T>) return to_f32(*p);
    else return (float)*p;
}
template <class T>
__device__ __forceinline__ T st_from_f32(float v) {
    if constexpr (is_half_v<T>) return from_f32<T>(v);
    else return (T)v;
}
template <class T>
__device__ __forceinline__ float up(T v) {
    if constexpr (is_half_v<T>) return to_f32(v);
    else return (float)v;
}
template <class T>
__device__ __forceinline__ float gelu_fwd(float x) {
    return gelu_f32_fast(x);  // the same function cuda_gelu_<T> evaluates
}

// u = round(z + b), a = round(gelu(u)); `a` may be NULL (bias add only).  The sum is rounded to
// T before the activation, exactly as the two separate ops would.
template <class T>
__global__ void __launch_bounds__(kFusedThreads) bias_gelu_kernel(const T* __restrict__ z, const T* __restrict__ bias, T* __restrict__ u,
                                                                 T* __restrict__ a, uint64_t n) {
    constexpr int VEC = 16 / sizeof(T);
    const float b = ld_scalar_f32(bias);
    const uint64_t nvec = n / VEC;
    const uint64_t stride = (uint64_t)gridDim.x * kFusedThreads;
    for (uint64_t v = (uint64_t)blockIdx.x * kFusedThreads + threadIdx.x; v < nvec; v += stride) {
        Vec<T, VEC> zi = *reinterpret_cast<const Vec<T, VEC>*>(z + v * VEC), uo, ao;
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            uo.v[j] = st_from_f32<T>(up(zi.v[j]) + b);
            ao.v[j] = st_from_f32<T>(gelu_fwd<T>(up(uo.v[j])));
        }
        *reinterpret_cast<Vec<T, VEC>*>(u + v * VEC) = uo;
        if (a) *reinterpret_cast<Vec<T, VEC>*>(a + v * VEC) = ao;
    }
    if (blockIdx.x == 0)
        for (uint64_t i = nvec * VEC + threadIdx.x; i < n; i += kFusedThreads) {
            T uu = st_from_f32<T>(up(z[i]) + b);
            u[i] = uu;
            if (a) a[i] = st_from_f32<T>(gelu_fwd<T>(up(uu)));
        }
}

__device__ __forceinline__ float gelu_grad_f32(float x) {
    const float s = 0.7978845608028654f, c = 0.044715f;
    const float x2 = x * x;
    const float t = s * (x + c * x2 * x);
    // tanh(t) = 1 - 2 / (1 + exp(2t)); sech^2 = 1 - tanh^2
    const float e = __expf(2.0f * t);
    const float th = 1.0f - __fdividef(2.0f, 1.0f + e);
    const float sech2 = 1.0f - th * th;
    return 0.5f * (1.0f + th) + 0.5f * x * sech2 * s * (1.0f + 3.0f * c * x2);
}

template <class T>
__global__ void __launch_bounds__(kFusedThreads) gelu_backward_kernel(const T* __restrict__ dy, const T* __restrict__ u, T* __restrict__ du,
                                                                     uint64_t n) {
    constexpr int VEC = 16 / sizeof(T);
    const uint64_t nvec = n / VEC;
    const uint64_t stride = (uint64_t)gridDim.x * kFusedThreads;
    for (uint64_t v = (uint64_t)blockIdx.x * kFusedThreads + threadIdx.x; v < nvec; v += stride) {
        Vec<T, VEC> g = *reinterpret_cast<const Vec<T, VEC>*>(dy + v * VEC), x = *reinterpret_cast<const Vec<T, VEC>*>(u + v * VEC), o;
#pragma unroll
        for (int j = 0; j < VEC; j++) o.v[j] = st_from_f32<T>(up(g.v[j]) * gelu_grad_f32(up(x.v[j])));
        *reinterpret_cast<Vec<T, VEC>*>(du + v * VEC) = o;
    }
    if (blockIdx.x == 0)
        for (uint64_t i = nvec * VEC + threadIdx.x; i < n; i += kFusedThreads) du[i] = st_from_f32<T>(up(dy[i]) * gelu_grad_f32(up(u[i])));
}

// Pass 1: grad = 2 (p - t) / n, per-block partial sums of (p - t)^2 into `partial`.
template <class T>
__global__ void __launch_bounds__(kFusedThreads) mse_kernel(const T* __restrict__ p, const T* __restrict__ t, T* __restrict__ grad,
                                                           float* __restrict__ partial, uint64_t n, float two_over_n) {
    constexpr int VEC = 16 / sizeof(T);
    const uint64_t nvec = n / VEC;
    const uint64_t stride = (uint64_t)gridDim.x * kFusedThreads;
    float acc = 0.0f;
    for (uint64_t v = (uint64_t)blockIdx.x * kFusedThreads + threadIdx.x; v < nvec; v += stride) {
        Vec<T, VEC> a = *reinterpret_cast<const Vec<T, VEC>*>(p + v * VEC), b = *reinterpret_cast<const Vec<T, VEC>*>(t + v * VEC), o;
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            // the difference is rounded to T first, as the separate sub op would
            float d = up(st_from_f32<T>(up(a.v[j]) - up(b.v[j])));
            acc += d * d;
            o.v[j] = st_from_f32<T>(d * two_over_n);
        }
        *reinterpret_cast<Vec<T, VEC>*>(grad + v * VEC) = o;
    }
    if (blockIdx.x == 0)
        for (uint64_t i = nvec * VEC + threadIdx.x; i < n; i += kFusedThreads) {
            float d = up(st_from_f32<T>(up(p[i]) - up(t[i])));
            acc += d * d;
            grad[i] = st_from_f32<T>(d * two_over_n);
        }
    __shared__ float warp_part[kFusedThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < kFusedThreads / 32 ? warp_part[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (threadIdx.x == 0) partial[blockIdx.x] = v;
    }
}
// Pass 2: one block folds the partials in a fixed order.
__global__ void __launch_bounds__(kFusedThreads) mse_finish_kernel(const float* __restrict__ partial, int count, float inv_n, float* __restrict__ loss) {
    __shared__ float sm[kFusedThreads];
    float acc = 0.0f;
    for (int i = threadIdx.x; i < count; i += kFusedThreads) acc += partial[i];
    sm[threadIdx.x] = acc;
    __syncthreads();
    for (int o = kFusedThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *loss = sm[0] * inv_n;
}

template <class T>
__global__ void __launch_bounds__(kFusedThreads) sgd_kernel(float* __restrict__ w32, const T* __restrict__ g, T* __restrict__ w16, uint64_t n,
                                                           float step) {
    constexpr int VEC = 16 / sizeof(T);  // elements per 16-byte vector of the gradient; w32 moves as VEC floats
    const uint64_t nvec = n / VEC;
    const uint64_t stride = (uint64_t)gridDim.x * kFusedThreads;
    for (uint64_t v = (uint64_t)blockIdx.x * kFusedThreads + threadIdx.x; v < nvec; v += stride) {
        Vec<T, VEC> gi = *reinterpret_cast<const Vec<T, VEC>*>(g + v * VEC), wo;
        // the master weights are promised 16-byte aligned only: move them as float4 quads, never as one 32-byte access
        float4 w[VEC / 4];
#pragma unroll
        for (int q = 0; q < VEC / 4; q++) w[q] = *reinterpret_cast<const float4*>(w32 + v * VEC + 4 * q);
#pragma unroll
        for (int q = 0; q < VEC / 4; q++) {
            w[q].x = w[q].x - step * up(gi.v[4 * q + 0]);
            w[q].y = w[q].y - step * up(gi.v[4 * q + 1]);
            w[q].z = w[q].z - step * up(gi.v[4 * q + 2]);
            w[q].w = w[q].w - step * up(gi.v[4 * q + 3]);
            wo.v[4 * q + 0] = st_from_f32<T>(w[q].x);
            wo.v[4 * q + 1] = st_from_f32<T>(w[q].y);
            wo.v[4 * q + 2] = st_from_f32<T>(w[q].z);
            wo.v[4 * q + 3] = st_from_f32<T>(w[q].w);
        }
#pragma unroll
        for (int q = 0; q < VEC / 4; q++) *reinterpret_cast<float4*>(w32 + v * VEC + 4 * q) = w[q];
        *reinterpret_cast<Vec<T, VEC>*>(w16 + v * VEC) = wo;
    }
    if (blockIdx.x == 0)
        for (uint64_t i = nvec * VEC + threadIdx.x; i < n; i += kFusedThreads) {
            float w = w32[i] - step * up(g[i]);
            w32[i] = w;
            w16[i] = st_from_f32<T>(w);
        }
}

static unsigned fused_grid(uint64_t n, int vec) {
    uint64_t blocks = (n / vec + kFusedThreads * 4 - 1) / (kFusedThreads * 4);
    uint64_t cap = (uint64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    return blocks ? (unsigned)blocks : 1u;
}
static bool aligned16(const void* p) { return ((uintptr_t)p) % 16 == 0; }

template <class T>
void bias_gelu_launch(size_t n, const T* z, const T* bias, T* u, T* a, const char* where) {
    if (!n) return;
    if (!aligned16(z) || !aligned16(u) || (a && !aligned16(a))) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    bias_gelu_kernel<T><<<fused_grid(n, 16 / sizeof(T)), kFusedThreads, 0, ctx().stream>>>(z, bias, u, a, n);
    check_launch(where);
}
template <class T>
void gelu_backward_launch(size_t n, const T* dy, const T* u, T* du, const char* where) {
    if (!n) return;
    if (!aligned16(dy) || !aligned16(u) || !aligned16(du)) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    gelu_backward_kernel<T><<<fused_grid(n, 16 / sizeof(T)), kFusedThreads, 0, ctx().stream>>>(dy, u, du, n);
    check_launch(where);
}
template <class T>
void mse_launch(size_t n, const T* p, const T* t, T* grad, float* loss, const char* where) {
    if (!n) return;
    if (!aligned16(p) || !aligned16(t) || !aligned16(grad)) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    unsigned blocks = fused_grid(n, 16 / sizeof(T));
    float* partial = static_cast<float*>(scratch(sizeof(float) * blocks));
    if (!partial) return;
    mse_kernel<T><<<blocks, kFusedThreads, 0, ctx().stream>>>(p, t, grad, partial, n, 2.0f / (float)n);
    mse_finish_kernel<<<1, kFusedThreads, 0, ctx().stream>>>(partial, (int)blocks, 1.0f / (float)n, loss);
    check_launch(where);
}
template <class T>
void sgd_launch(size_t n, float* w32, const T* g, T* w16, float lr, float grad_scale, const char* where) {
    if (!n) return;
    if (!aligned16(w32) || !aligned16(g) || !aligned16(w16)) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    sgd_kernel<T><<<fused_grid(n, 16 / sizeof(T)), kFusedThreads, 0, ctx().stream>>>(w32, g, w16, n, lr * grad_scale);
    check_launch(where);
}

}  // namespace mx

#define DEF_FUSED(T)                                                                                                                    \
    void mx_bias_gelu_##T(size_t n, const mx_##T* z, const mx_##T* bias, mx_##T* u, mx_##T* a) {                                        \
        mx::bias_gelu_launch<mx_##T>(n, z, bias, u, a, "mx_bias_gelu_" #T);                                                             \
    }                                                                                                                                   \
    void mx_gelu_backward_##T(size_t n, const mx_##T* dy, const mx_##T* u, mx_##T* du) {                                                \
        mx::gelu_backward_launch<mx_##T>(n, dy, u, du, "mx_gelu_backward_" #T);                                                         \
    }                                                                                                                                   \
    void mx_mse_loss_grad_##T(size_t n, const mx_##T* pred, const mx_##T* target, mx_##T* grad, float* loss) {                          \
        mx::mse_launch<mx_##T>(n, pred, target, grad, loss, "mx_mse_loss_grad_" #T);                                                    \
    }                                                                                                                                   \
    void mx_sgd_update_##T(size_t n, float* w32, const mx_##T* grad, mx_##T* w16, float lr, float grad_scale) {                         \
        mx::sgd_launch<mx_##T>(n, w32, grad, w16, lr, grad_scale, "mx_sgd_update_" #T);                                                 \
    }

// Linear forward in one call: u[rows, out] = x[rows, in] . w[out, in]^T + bias (one element), act = gelu(u) (act may be NULL).
// Large bf16 / f16 layers run the product on the tensor cores with bias and activation in its epilogue; any other
// shape runs cuda_matmul into u followed by the in-place bias / activation pass.  Both give the bits of the three separate
// ops of crates/maidenx_nn/src/layers/linear.rs:60-81 followed by gelu.
#define DEF_LINEAR(T, IS_BF16)                                                                                                          \
    void mx_linear_bias_gelu_##T(size_t rows, size_t in_features, size_t out_features, const mx_##T* x, const mx_##T* w, const mx_##T* bias, \
                                 mx_##T* u, mx_##T* act) {                                                                              \
        if (!rows || !in_features || !out_features) return;                                                                             \
        if (mx::tc_linear_bias_act(IS_BF16, rows, in_features, out_features, x, w, bias, u, act, "mx_linear_bias_gelu_" #T)) return;       \
        const size_t meta[] = {2, 2, 2, rows, out_features, rows, in_features, in_features, out_features, in_features, 1, 1, in_features, 0, 0}; \
        cuda_matmul_##T(rows * out_features, meta, x, w, u);                                                                            \
        mx::bias_gelu_launch<mx_##T>(rows * out_features, u, bias, u, act, "mx_linear_bias_gelu_" #T);                                    \
    }

extern "C" {
DEF_FUSED(bf16)
DEF_FUSED(f16)
DEF_FUSED(f32)
DEF_LINEAR(bf16, true)
DEF_LINEAR(f16, false)
}
