// MLP training step composed from the op layer: the data-parallel workload of the benchmark.
//
// The model is the reference's recipe at width D: L x [Linear(D -> D) with a scalar bias
// (crates/maidenx_nn/src/layers/linear.rs:25-81), GELU between layers], MSE loss
// (crates/maidenx_nn/src/losses/mse.rs:21-29), SGD (crates/maidenx_nn/src/optimizers/sgd.rs:17-26),
// in bf16 or f16 with f32 master weights.  Every matrix product goes through the C-ABI entry
// point cuda_matmul_<T> with the metadata the reference's tensor layer would build:
//   forward   z = a_prev . W^T        B is the transposed view of W [D_out, D_in] (strides [1, D_in])
//   grad in   da_prev = du . W        contiguous operands
//   grad W    dW = du^T . a_prev      A is the transposed view of du (strides [1, D_out]): the
//                                     "two strided matmuls" of the reference's graph-mode backward
//                                     (crates/maidenx_tensor_v2/src/ops/_try_matmul.rs:98-140)
// (dX and dW are the mathematically correct products; the reference's eager matmul_backward,
// which ignores the strides of the transposed weight view, is exercised separately by the
// parity tests.)  Elementwise passes use the fused mx_* kernels; the bias gradient is a
// cuda_sum_<T> over du.
//
// The step is split so that a data-parallel driver can overlap the gradient all-reduce of layer
// l with the backward of layer l-1: forward, loss_backward, backward_layer(l), sgd_layer(l).
#include <cmath>
#include <cstring>
#include <vector>

#include "abi_common.cuh"

extern "C" {
void mx_bias_gelu_bf16(size_t, const mx_bf16*, const mx_bf16*, mx_bf16*, mx_bf16*);
void mx_bias_gelu_f16(size_t, const mx_f16*, const mx_f16*, mx_f16*, mx_f16*);
void mx_gelu_backward_bf16(size_t, const mx_bf16*, const mx_bf16*, mx_bf16*);
void mx_gelu_backward_f16(size_t, const mx_f16*, const mx_f16*, mx_f16*);
void mx_mse_loss_grad_bf16(size_t, const mx_bf16*, const mx_bf16*, mx_bf16*, float*);
void mx_mse_loss_grad_f16(size_t, const mx_f16*, const mx_f16*, mx_f16*, float*);
void mx_sgd_update_bf16(size_t, float*, const mx_bf16*, mx_bf16*, float, float);
void mx_sgd_update_f16(size_t, float*, const mx_f16*, mx_f16*, float, float);
}

namespace mx {

struct Mlp {
    int layers = 0;
    size_t dim = 0, batch = 0;
    bool is_bf16 = true;
    // per layer
    std::vector<float*> w32, b32;        // f32 master copies [dim*dim], [1]
    std::vector<uint16_t*> w16, b16;     // 16-bit working copies
    std::vector<uint16_t*> gw, gb;       // gradients (16-bit): [dim*dim], [1]
    std::vector<uint16_t*> u, a;         // pre-activation (z + b) and activation, [batch*dim]; a[L-1] unused
    uint16_t* z = nullptr;               // GEMM output before the bias add (reused by every layer)
    uint16_t* d_act = nullptr;           // gradient w.r.t. the current layer's output
    uint16_t* d_pre = nullptr;           // gradient w.r.t. the current layer's pre-activation
    const uint16_t* x = nullptr;         // input batch of the current step
    float* loss = nullptr;               // device scalar
    std::vector<void*> owned;
};

static void* dmalloc(Mlp* m, size_t bytes) {
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        set_error(kErrCuda, (int)cudaGetLastError(), "mx_mlp_create");
        return nullptr;
    }
    m->owned.push_back(p);
    return p;
}

// counter-based generator shared with the host-side parity code: SplitMix64 of (seed, index)
__host__ __device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__host__ __device__ inline float uniform_pm(uint64_t seed, uint64_t i, float bound) {
    uint64_t r = splitmix64(seed * 0x100000001B3ull + i);
    float u = (float)(r >> 40) * (1.0f / 16777216.0f);  // [0, 1)
    return (2.0f * u - 1.0f) * bound;
}
template <class T>
__global__ void init_weights_kernel(float* w32, T* w16, uint64_t n, uint64_t seed, float bound) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float v = uniform_pm(seed, i, bound);
        w32[i] = v;
        w16[i] = from_f32<T>(v);
    }
}

template <class T>
static void matmul_call(size_t num_els, const size_t* meta, const T* a, const T* b, T* c);
template <>
void matmul_call<bf16>(size_t n, const size_t* m, const bf16* a, const bf16* b, bf16* c) { cuda_matmul_bf16(n, m, a, b, c); }
template <>
void matmul_call<f16>(size_t n, const size_t* m, const f16* a, const f16* b, f16* c) { cuda_matmul_f16(n, m, a, b, c); }

template <class T>
static void forward_t(Mlp* m, const T* x) {
    const size_t B = m->batch, D = m->dim;
    m->x = reinterpret_cast<const uint16_t*>(x);
    const T* prev = x;
    for (int l = 0; l < m->layers; l++) {
        // out [B, D], A [B, D] strides [D, 1], B = W^T view: shape [D, D] strides [1, D]
        const size_t meta[] = {2, 2, 2, B, D, B, D, D, D, D, 1, 1, D, 0, 0};
        matmul_call<T>(B * D, meta, prev, reinterpret_cast<const T*>(m->w16[l]), reinterpret_cast<T*>(m->z));
        const bool last = l == m->layers - 1;
        T* act = last ? nullptr : reinterpret_cast<T*>(m->a[l]);
        if constexpr (std::is_same<T, bf16>::value)
            mx_bias_gelu_bf16(B * D, reinterpret_cast<const T*>(m->z), reinterpret_cast<const T*>(m->b16[l]), reinterpret_cast<T*>(m->u[l]), act);
        else
            mx_bias_gelu_f16(B * D, reinterpret_cast<const T*>(m->z), reinterpret_cast<const T*>(m->b16[l]), reinterpret_cast<T*>(m->u[l]), act);
        prev = act;
    }
}

template <class T>
static void loss_backward_t(Mlp* m, const T* y) {
    const size_t n = m->batch * m->dim;
    const T* pred = reinterpret_cast<const T*>(m->u[m->layers - 1]);
    if constexpr (std::is_same<T, bf16>::value) mx_mse_loss_grad_bf16(n, pred, y, reinterpret_cast<T*>(m->d_pre), m->loss);
    else mx_mse_loss_grad_f16(n, pred, y, reinterpret_cast<T*>(m->d_pre), m->loss);
}

template <class T>
static void backward_layer_t(Mlp* m, int l) {
    const size_t B = m->batch, D = m->dim, n = B * D;
    T* du = reinterpret_cast<T*>(m->d_pre);
    if (l != m->layers - 1) {
        // d_act holds the gradient w.r.t. a[l]; turn it into the gradient w.r.t. u[l]
        if constexpr (std::is_same<T, bf16>::value)
            mx_gelu_backward_bf16(n, reinterpret_cast<const T*>(m->d_act), reinterpret_cast<const T*>(m->u[l]), du);
        else
            mx_gelu_backward_f16(n, reinterpret_cast<const T*>(m->d_act), reinterpret_cast<const T*>(m->u[l]), du);
    }
    // bias gradient: sum of du over all elements (the scalar bias broadcasts over the whole output)
    {
        const size_t meta[] = {n, 1, n, 1, 0};  // dims | strides | red_len | red_stride | offset
        if constexpr (std::is_same<T, bf16>::value) cuda_sum_bf16(n, 1, 1, meta, du, reinterpret_cast<T*>(m->gb[l]));
        else cuda_sum_f16(n, 1, 1, meta, du, reinterpret_cast<T*>(m->gb[l]));
    }
    const T* a_prev = l == 0 ? reinterpret_cast<const T*>(m->x) : reinterpret_cast<const T*>(m->a[l - 1]);
    // dW [D_out, D_in] = du^T . a_prev: A = transposed view of du (shape [D, B], strides [1, D]), B = a_prev [B, D]
    {
        const size_t meta[] = {2, 2, 2, D, D, D, B, B, D, 1, D, D, 1, 0, 0};
        matmul_call<T>(D * D, meta, du, a_prev, reinterpret_cast<T*>(m->gw[l]));
    }
    // gradient for the layer below: da_prev [B, D_in] = du [B, D_out] . W [D_out, D_in]
    if (l > 0) {
        const size_t meta[] = {2, 2, 2, B, D, B, D, D, D, D, 1, D, 1, 0, 0};
        matmul_call<T>(n, meta, du, reinterpret_cast<const T*>(m->w16[l]), reinterpret_cast<T*>(m->d_act));
    }
}

template <class T>
static void sgd_layer_t(Mlp* m, int l, float lr, float grad_scale) {
    const size_t D = m->dim;
    if constexpr (std::is_same<T, bf16>::value) {
        mx_sgd_update_bf16(D * D, m->w32[l], reinterpret_cast<const T*>(m->gw[l]), reinterpret_cast<T*>(m->w16[l]), lr, grad_scale);
        mx_sgd_update_bf16(1, m->b32[l], reinterpret_cast<const T*>(m->gb[l]), reinterpret_cast<T*>(m->b16[l]), lr, grad_scale);
    } else {
        mx_sgd_update_f16(D * D, m->w32[l], reinterpret_cast<const T*>(m->gw[l]), reinterpret_cast<T*>(m->w16[l]), lr, grad_scale);
        mx_sgd_update_f16(1, m->b32[l], reinterpret_cast<const T*>(m->gb[l]), reinterpret_cast<T*>(m->b16[l]), lr, grad_scale);
    }
}

}  // namespace mx

using namespace mx;

extern "C" {

// dtype: 0 = bf16, 1 = f16.  Weights are initialised U(-1/sqrt(dim), 1/sqrt(dim)) from `seed`
// (Kaiming-uniform with a = sqrt(5)), the scalar biases likewise; identical on every rank.
void* mx_mlp_create(int layers, size_t dim, size_t batch, int dtype, uint64_t seed) {
    if (layers <= 0 || dim == 0 || batch == 0 || (dtype != 0 && dtype != 1)) return nullptr;
    Mlp* m = new Mlp();
    m->layers = layers;
    m->dim = dim;
    m->batch = batch;
    m->is_bf16 = dtype == 0;
    const size_t wn = dim * dim, an = batch * dim;
    bool ok = true;
    for (int l = 0; l < layers && ok; l++) {
        // biases live in 256-byte slots so that every pointer handed to a vector kernel is aligned
        m->w32.push_back(static_cast<float*>(dmalloc(m, wn * 4)));
        m->b32.push_back(static_cast<float*>(dmalloc(m, 256)));
        m->w16.push_back(static_cast<uint16_t*>(dmalloc(m, wn * 2)));
        m->b16.push_back(static_cast<uint16_t*>(dmalloc(m, 256)));
        m->gw.push_back(static_cast<uint16_t*>(dmalloc(m, wn * 2)));
        m->gb.push_back(static_cast<uint16_t*>(dmalloc(m, 256)));
        m->u.push_back(static_cast<uint16_t*>(dmalloc(m, an * 2)));
        m->a.push_back(l == layers - 1 ? nullptr : static_cast<uint16_t*>(dmalloc(m, an * 2)));
        ok = m->w32[l] && m->b32[l] && m->w16[l] && m->b16[l] && m->gw[l] && m->gb[l] && m->u[l] && (l == layers - 1 || m->a[l]);
    }
    m->z = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->d_act = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->d_pre = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->loss = static_cast<float*>(dmalloc(m, 256));
    ok = ok && m->z && m->d_act && m->d_pre && m->loss;
    if (!ok) {
        for (void* p : m->owned) cudaFree(p);
        delete m;
        return nullptr;
    }
    const float bound = 1.0f / std::sqrt((float)dim);
    for (int l = 0; l < layers; l++) {
        cudaMemsetAsync(m->b32[l], 0, 256, ctx().stream);
        cudaMemsetAsync(m->b16[l], 0, 256, ctx().stream);
        cudaMemsetAsync(m->gb[l], 0, 256, ctx().stream);
        if (m->is_bf16) {
            init_weights_kernel<bf16><<<1024, 256, 0, ctx().stream>>>(m->w32[l], reinterpret_cast<bf16*>(m->w16[l]), wn, seed + 2 * l, bound);
            init_weights_kernel<bf16><<<1, 32, 0, ctx().stream>>>(m->b32[l], reinterpret_cast<bf16*>(m->b16[l]), 1, seed + 2 * l + 1, bound);
        } else {
            init_weights_kernel<f16><<<1024, 256, 0, ctx().stream>>>(m->w32[l], reinterpret_cast<f16*>(m->w16[l]), wn, seed + 2 * l, bound);
            init_weights_kernel<f16><<<1, 32, 0, ctx().stream>>>(m->b32[l], reinterpret_cast<f16*>(m->b16[l]), 1, seed + 2 * l + 1, bound);
        }
    }
    check_launch("mx_mlp_create");
    return m;
}

void mx_mlp_destroy(void* h) {
    Mlp* m = static_cast<Mlp*>(h);
    if (!m) return;
    for (void* p : m->owned) cudaFree(p);
    delete m;
}

void mx_mlp_forward(void* h, const void* x) {
    Mlp* m = static_cast<Mlp*>(h);
    if (m->is_bf16) forward_t<bf16>(m, static_cast<const bf16*>(x));
    else forward_t<f16>(m, static_cast<const f16*>(x));
}
void mx_mlp_loss_backward(void* h, const void* y) {
    Mlp* m = static_cast<Mlp*>(h);
    if (m->is_bf16) loss_backward_t<bf16>(m, static_cast<const bf16*>(y));
    else loss_backward_t<f16>(m, static_cast<const f16*>(y));
}
void mx_mlp_backward_layer(void* h, int l) {
    Mlp* m = static_cast<Mlp*>(h);
    if (l < 0 || l >= m->layers) return;
    if (m->is_bf16) backward_layer_t<bf16>(m, l);
    else backward_layer_t<f16>(m, l);
}
void mx_mlp_sgd_layer(void* h, int l, float lr, float grad_scale) {
    Mlp* m = static_cast<Mlp*>(h);
    if (l < 0 || l >= m->layers) return;
    if (m->is_bf16) sgd_layer_t<bf16>(m, l, lr, grad_scale);
    else sgd_layer_t<f16>(m, l, lr, grad_scale);
}
// Device pointers for the data-parallel driver (gradient all-reduce) and for parity checks.
void* mx_mlp_weight_grad(void* h, int l) { return static_cast<Mlp*>(h)->gw[l]; }
void* mx_mlp_bias_grad(void* h, int l) { return static_cast<Mlp*>(h)->gb[l]; }
float* mx_mlp_master_weight(void* h, int l) { return static_cast<Mlp*>(h)->w32[l]; }
float* mx_mlp_master_bias(void* h, int l) { return static_cast<Mlp*>(h)->b32[l]; }
void* mx_mlp_weight(void* h, int l) { return static_cast<Mlp*>(h)->w16[l]; }
void* mx_mlp_output(void* h) { return static_cast<Mlp*>(h)->u[static_cast<Mlp*>(h)->layers - 1]; }
float* mx_mlp_loss_ptr(void* h) { return static_cast<Mlp*>(h)->loss; }
// Copies the loss of the last loss_backward to the host (synchronises the stream).
float mx_mlp_loss(void* h) {
    Mlp* m = static_cast<Mlp*>(h);
    float v = NAN;
    cudaMemcpyAsync(&v, m->loss, sizeof(float), cudaMemcpyDeviceToHost, ctx().stream);
    cudaStreamSynchronize(ctx().stream);
    return v;
}

}  // extern "C"
