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
#include <cstdio>
#include <cstdlib>
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
void mx_linear_bias_gelu_bf16(size_t, size_t, size_t, const mx_bf16*, const mx_bf16*, const mx_bf16*, mx_bf16*, mx_bf16*);
void mx_linear_bias_gelu_f16(size_t, size_t, size_t, const mx_f16*, const mx_f16*, const mx_f16*, mx_f16*, mx_f16*);
void mx_sgd_update_bf16(size_t, float*, const mx_bf16*, mx_bf16*, float, float);
void mx_sgd_update_f16(size_t, float*, const mx_f16*, mx_f16*, float, float);
void mx_dp_barrier(void* const*, size_t, int, int, uint32_t, uint32_t*, void*);
void mx_dp_reduce_sgd(int, void* const*, void*, const void* const*, int, int, size_t, size_t, size_t, float*, size_t, size_t, float*, void*, float, int, void*);
void mx_mlp_destroy(void*);
}

namespace mx {

constexpr int kMlpMaxWorld = 16;

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
    uint16_t* du[2] = {nullptr, nullptr};  // gradient w.r.t. a layer's pre-activation; layer l uses du[l & 1], so the
                                         // data-parallel step can finish layer 0 before it computes layer 1's weight gradient
    const uint16_t* x = nullptr;         // input batch of the current step
    float* loss = nullptr;               // device scalar
    std::vector<void*> owned;
    // data-parallel mode over peer-mapped arenas (dp_sync.cu); world == 1 and dp == false otherwise
    bool dp = false;
    int rank = 0, world = 1;
    void* peer[kMlpMaxWorld] = {nullptr};  // every rank's arena as mapped here; peer[rank] is the local one
    void* mc = nullptr;                    // multicast address of the arenas, or NULL
    std::vector<size_t> gw_off, w_off, gb_off;  // byte offsets of a layer's buffers inside every arena
    size_t shard_begin = 0, shard_elems = 0;    // this rank's slice of every weight matrix (elements)
    cudaStream_t side = nullptr;                // the exchange runs here, beside the backward of the layers below
    std::vector<cudaEvent_t> ev_grad, ev_done;  // per layer: gradient ready (main stream) / new weights landed (side stream)
    uint32_t epoch = 0;                         // barrier counter, the same sequence on every rank
    uint32_t* dp_err = nullptr;                 // device word: 0, or 1 + the peer a barrier gave up on
    // copy-engine exchange: the peers' gradient shards are pulled into `staging`, summed locally, and the new
    // weights pushed back with plain device-to-device copies, so no SM ever waits on NVLink
    bool copy_engines = false;
    int exclusive_sms = 0;  // > 0: the multimem exchange kernel keeps this many SMs to itself and the step's GEMMs use the rest
    void* staging[kMlpMaxWorld] = {nullptr};
};

// Arena layout: [flags, 4 KiB][per layer: weight gradient | 16-bit weights | bias-gradient slot], each 4 KiB aligned.
static size_t arena_align(size_t b) { return (b + 4095) / 4096 * 4096; }
static size_t arena_layer_bytes(size_t dim) { return 2 * arena_align(dim * dim * 2) + 4096; }

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
// Fills the 16-bit working copy [0, n) (when w16 != NULL) and the f32 master values of
// [m_begin, m_begin + m_count) into w32[0 .. m_count): the master copy may be just a shard.
template <class T>
__global__ void init_weights_kernel(float* w32, uint64_t m_begin, uint64_t m_count, T* w16, uint64_t n, uint64_t seed, float bound) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float v = uniform_pm(seed, i, bound);
        if (i >= m_begin && i - m_begin < m_count) w32[i - m_begin] = v;
        if (w16) w16[i] = from_f32<T>(v);
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
        // the layer's weights of the previous step must have landed: from every rank in data-parallel mode, from the
        // side stream's optimizer update in mx_mlp_train_step (an event that was never recorded does not block)
        if (l < (int)m->ev_done.size()) cudaStreamWaitEvent(ctx().stream, m->ev_done[l], 0);
        // u[l] = prev . W^T + bias, a[l] = gelu(u[l]): the product with bias and activation in its epilogue
        const bool last = l == m->layers - 1;
        T* act = last ? nullptr : reinterpret_cast<T*>(m->a[l]);
        if constexpr (std::is_same<T, bf16>::value)
            mx_linear_bias_gelu_bf16(B, D, D, prev, reinterpret_cast<const T*>(m->w16[l]), reinterpret_cast<const T*>(m->b16[l]), reinterpret_cast<T*>(m->u[l]), act);
        else
            mx_linear_bias_gelu_f16(B, D, D, prev, reinterpret_cast<const T*>(m->w16[l]), reinterpret_cast<const T*>(m->b16[l]), reinterpret_cast<T*>(m->u[l]), act);
        prev = act;
    }
}

template <class T>
static void loss_backward_t(Mlp* m, const T* y) {
    const size_t n = m->batch * m->dim;
    const T* pred = reinterpret_cast<const T*>(m->u[m->layers - 1]);
    if constexpr (std::is_same<T, bf16>::value) mx_mse_loss_grad_bf16(n, pred, y, reinterpret_cast<T*>(m->du[(m->layers - 1) & 1]), m->loss);
    else mx_mse_loss_grad_f16(n, pred, y, reinterpret_cast<T*>(m->du[(m->layers - 1) & 1]), m->loss);
}

// Backward of layer l, first part: the gradient w.r.t. the pre-activation, the bias gradient, and the gradient
// handed to the layer below (which reads W[l]).
template <class T>
static void backward_input_t(Mlp* m, int l) {
    const size_t B = m->batch, D = m->dim, n = B * D;
    T* du = reinterpret_cast<T*>(m->du[l & 1]);
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
    // gradient for the layer below: da_prev [B, D_in] = du [B, D_out] . W [D_out, D_in]
    if (l > 0) {
        const size_t meta[] = {2, 2, 2, B, D, B, D, D, D, D, 1, D, 1, 0, 0};
        matmul_call<T>(n, meta, du, reinterpret_cast<const T*>(m->w16[l]), reinterpret_cast<T*>(m->d_act));
    }
}

// Second part: dW [D_out, D_in] = du^T . a_prev: A = transposed view of du (shape [D, B], strides [1, D]),
// B = a_prev [B, D].  Queued after the first part, so "dW[l] done" implies "W[l] no longer needed" - the
// data-parallel exchange overwrites W[l] as soon as every rank has its dW[l].
template <class T>
static void backward_weight_t(Mlp* m, int l) {
    const size_t B = m->batch, D = m->dim;
    const T* du = reinterpret_cast<const T*>(m->du[l & 1]);
    const T* a_prev = l == 0 ? reinterpret_cast<const T*>(m->x) : reinterpret_cast<const T*>(m->a[l - 1]);
    const size_t meta[] = {2, 2, 2, D, D, D, B, B, D, 1, D, D, 1, 0, 0};
    matmul_call<T>(D * D, meta, du, a_prev, reinterpret_cast<T*>(m->gw[l]));
}

template <class T>
static void backward_layer_t(Mlp* m, int l) {
    backward_input_t<T>(m, l);
    backward_weight_t<T>(m, l);
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

namespace mx {

// Shared by mx_mlp_create and mx_mlp_create_dp.  peer == NULL: single-device engine.
static Mlp* mlp_create_impl(int layers, size_t dim, size_t batch, int dtype, uint64_t seed, int rank, int world, void* const* peer, void* multicast) {
    const char* where = peer ? "mx_mlp_create_dp" : "mx_mlp_create";
    if (layers <= 0 || dim == 0 || batch == 0 || (dtype != 0 && dtype != 1)) return nullptr;
    const size_t wn = dim * dim, an = batch * dim;
    if (peer && (world < 1 || world > kMlpMaxWorld || rank < 0 || rank >= world || wn % (8 * (size_t)world) != 0)) {
        set_error(kErrBadMetadata, 0, where);
        return nullptr;
    }
    Mlp* m = new Mlp();
    m->layers = layers;
    m->dim = dim;
    m->batch = batch;
    m->is_bf16 = dtype == 0;
    m->dp = peer != nullptr;
    m->rank = peer ? rank : 0;
    m->world = peer ? world : 1;
    m->shard_elems = wn / (size_t)m->world;
    m->shard_begin = m->shard_elems * (size_t)m->rank;
    char* arena = nullptr;
    if (peer) {
        for (int p = 0; p < world; p++) m->peer[p] = peer[p];
        m->mc = multicast;
        arena = static_cast<char*>(peer[rank]);
    }
    bool ok = true;
    for (int l = 0; l < layers && ok; l++) {
        // biases live in 256-byte slots so that every pointer handed to a vector kernel is aligned
        m->w32.push_back(static_cast<float*>(dmalloc(m, m->shard_elems * 4)));  // master weights: only this rank's shard
        m->b32.push_back(static_cast<float*>(dmalloc(m, 256)));
        m->b16.push_back(static_cast<uint16_t*>(dmalloc(m, 256)));
        if (peer) {
            const size_t base = 4096 + (size_t)l * arena_layer_bytes(dim);
            m->gw_off.push_back(base);
            m->w_off.push_back(base + arena_align(wn * 2));
            m->gb_off.push_back(base + 2 * arena_align(wn * 2));
            m->gw.push_back(reinterpret_cast<uint16_t*>(arena + m->gw_off[l]));
            m->w16.push_back(reinterpret_cast<uint16_t*>(arena + m->w_off[l]));
            m->gb.push_back(reinterpret_cast<uint16_t*>(arena + m->gb_off[l]));
        } else {
            m->w16.push_back(static_cast<uint16_t*>(dmalloc(m, wn * 2)));
            m->gw.push_back(static_cast<uint16_t*>(dmalloc(m, wn * 2)));
            m->gb.push_back(static_cast<uint16_t*>(dmalloc(m, 256)));
        }
        m->u.push_back(static_cast<uint16_t*>(dmalloc(m, an * 2)));
        m->a.push_back(l == layers - 1 ? nullptr : static_cast<uint16_t*>(dmalloc(m, an * 2)));
        ok = m->w32[l] && m->b32[l] && m->w16[l] && m->b16[l] && m->gw[l] && m->gb[l] && m->u[l] && (l == layers - 1 || m->a[l]);
    }
    m->z = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->d_act = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->du[0] = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->du[1] = static_cast<uint16_t*>(dmalloc(m, an * 2));
    m->loss = static_cast<float*>(dmalloc(m, 256));
    m->dp_err = static_cast<uint32_t*>(dmalloc(m, 256));
    ok = ok && m->z && m->d_act && m->du[0] && m->du[1] && m->loss && m->dp_err;
    if (ok) {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        ok = cudaStreamCreateWithPriority(&m->side, cudaStreamNonBlocking, hi) == cudaSuccess;
        for (int l = 0; l < layers && ok; l++) {
            cudaEvent_t e1 = nullptr, e2 = nullptr;
            ok = cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) == cudaSuccess && cudaEventCreateWithFlags(&e2, cudaEventDisableTiming) == cudaSuccess;
            m->ev_grad.push_back(e1);
            m->ev_done.push_back(e2);
        }
    }
    if (!ok) {
        set_error(kErrCuda, (int)cudaGetLastError(), where);
        mx_mlp_destroy(m);
        return nullptr;
    }
    const float bound = 1.0f / std::sqrt((float)dim);
    cudaStream_t s = ctx().stream;
    cudaMemsetAsync(m->dp_err, 0, 256, s);
    for (int l = 0; l < layers; l++) {
        cudaMemsetAsync(m->b32[l], 0, 256, s);
        cudaMemsetAsync(m->b16[l], 0, 256, s);
        cudaMemsetAsync(m->gb[l], 0, 256, s);
        if (m->is_bf16) {
            init_weights_kernel<bf16><<<1024, 256, 0, s>>>(m->w32[l], m->shard_begin, m->shard_elems, reinterpret_cast<bf16*>(m->w16[l]), wn, seed + 2 * l, bound);
            init_weights_kernel<bf16><<<1, 32, 0, s>>>(m->b32[l], 0, 1, reinterpret_cast<bf16*>(m->b16[l]), 1, seed + 2 * l + 1, bound);
        } else {
            init_weights_kernel<f16><<<1024, 256, 0, s>>>(m->w32[l], m->shard_begin, m->shard_elems, reinterpret_cast<f16*>(m->w16[l]), wn, seed + 2 * l, bound);
            init_weights_kernel<f16><<<1, 32, 0, s>>>(m->b32[l], 0, 1, reinterpret_cast<f16*>(m->b16[l]), 1, seed + 2 * l + 1, bound);
        }
    }
    check_launch(where);
    return m;
}

}  // namespace mx

using namespace mx;

extern "C" {

// dtype: 0 = bf16, 1 = f16.  Weights are initialised U(-1/sqrt(dim), 1/sqrt(dim)) from `seed`
// (Kaiming-uniform with a = sqrt(5)), the scalar biases likewise; identical on every rank.
void* mx_mlp_create(int layers, size_t dim, size_t batch, int dtype, uint64_t seed) {
    return mlp_create_impl(layers, dim, batch, dtype, seed, 0, 1, nullptr, nullptr);
}

// Bytes of the peer-mapped arena every rank must provide to mx_mlp_create_dp.
size_t mx_mlp_dp_arena_bytes(int layers, size_t dim) { return 4096 + (size_t)(layers > 0 ? layers : 0) * arena_layer_bytes(dim); }

// Data-parallel engine.  peer_arenas[p]: rank p's arena (mx_mlp_dp_arena_bytes bytes, zero-filled,
// 4 KiB aligned) as mapped into this process; multicast_arena: the multicast address bound to all of
// them, or NULL (then the exchange uses peer loads and stores).  `batch` is this rank's share of the
// global batch.  Gradients, 16-bit weights and the barrier flags live in the arena; dim * dim must be
// a multiple of 8 * world.  The arenas must stay mapped until mx_mlp_destroy.
void* mx_mlp_create_dp(int layers, size_t dim, size_t batch, int dtype, uint64_t seed, int rank, int world, void* const* peer_arenas,
                       void* multicast_arena) {
    if (!peer_arenas) return nullptr;
    return mlp_create_impl(layers, dim, batch, dtype, seed, rank, world, peer_arenas, multicast_arena);
}

void mx_mlp_destroy(void* h) {
    Mlp* m = static_cast<Mlp*>(h);
    if (!m) return;
    if (m->side) {
        cudaStreamSynchronize(m->side);
        cudaStreamDestroy(m->side);
    }
    for (cudaEvent_t e : m->ev_grad) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : m->ev_done) if (e) cudaEventDestroy(e);
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
    if (m->dp) {  // the master weights are sharded: the update belongs to mx_mlp_train_step_dp
        set_error(kErrUnsupported, 0, "mx_mlp_sgd_layer");
        return;
    }
    if (m->is_bf16) sgd_layer_t<bf16>(m, l, lr, grad_scale);
    else sgd_layer_t<f16>(m, l, lr, grad_scale);
}
// One whole training step of the single-device engine.  The optimizer update of layer l is memory-bound and nothing
// below it in the backward pass needs its result, so it runs on the side stream beside the backward products of the
// layers below (which are bound by the tensor cores, not by HBM); the next forward waits, per layer, for that layer's
// update only.  Readers of the weights after the step call mx_mlp_dp_join (or synchronise the device).
void mx_mlp_train_step(void* h, const void* x, const void* y, float lr, float grad_scale) {
    Mlp* m = static_cast<Mlp*>(h);
    if (m->dp || !m->side) {
        set_error(kErrUnsupported, 0, "mx_mlp_train_step");
        return;
    }
    cudaStream_t main_stream = ctx().stream;
    mx_mlp_forward(h, x);
    mx_mlp_loss_backward(h, y);
    for (int l = m->layers - 1; l >= 0; l--) {
        mx_mlp_backward_layer(h, l);
        cudaEventRecord(m->ev_grad[l], main_stream);
        cudaStreamWaitEvent(m->side, m->ev_grad[l], 0);
        ctx().stream = m->side;
        if (m->is_bf16) sgd_layer_t<bf16>(m, l, lr, grad_scale);
        else sgd_layer_t<f16>(m, l, lr, grad_scale);
        ctx().stream = main_stream;
        cudaEventRecord(m->ev_done[l], m->side);
    }
    check_launch("mx_mlp_train_step");
}

// One whole data-parallel training step: forward, loss, backward, and per layer the fused
// gradient exchange + SGD update (dp_sync.cu) on a side stream, so that the exchange of layer l
// runs beside the backward of the layers below it.  `grad_scale` multiplies the summed gradient
// (1 / world for the mean over the global batch).  Every rank must make the same sequence of calls.
void mx_mlp_train_step_dp(void* h, const void* x, const void* y, float lr, float grad_scale) {
    Mlp* m = static_cast<Mlp*>(h);
    if (!m->dp) {
        set_error(kErrUnsupported, 0, "mx_mlp_train_step_dp");
        return;
    }
    cudaStream_t main_stream = ctx().stream;
    const int saved_limit = ctx().gemm_sm_limit;
    if (!m->copy_engines && m->mc && m->exclusive_sms > 0 && m->exclusive_sms < sm_count()) ctx().gemm_sm_limit = sm_count() - m->exclusive_sms;
    mx_mlp_forward(h, x);
    mx_mlp_loss_backward(h, y);
    const size_t flag_off = 0;
    // Exchange of layer l, queued on the side stream behind "dW[l] done".
    auto exchange = [&](int l) {
        cudaEventRecord(m->ev_grad[l], main_stream);
        cudaStreamWaitEvent(m->side, m->ev_grad[l], 0);
        mx_dp_barrier(m->peer, flag_off, m->rank, m->world, ++m->epoch, m->dp_err, m->side);
        const size_t shard_bytes = m->shard_elems * 2, shard_byte0 = m->shard_begin * 2;
        if (m->copy_engines) {
            // pull my shard of every peer's gradient, starting with the next rank so that no peer is asked by everyone at once
            for (int k = 1; k < m->world; k++) {
                const int p = (m->rank + k) % m->world;
                cudaMemcpyAsync(m->staging[p], static_cast<const char*>(m->peer[p]) + m->gw_off[l] + shard_byte0, shard_bytes, cudaMemcpyDeviceToDevice, m->side);
            }
            mx_dp_reduce_sgd(m->is_bf16 ? 0 : 1, m->peer, nullptr, m->staging, m->rank, m->world, m->gw_off[l], m->w_off[l], m->gb_off[l], m->w32[l],
                             m->shard_begin, m->shard_elems, m->b32[l], m->b16[l], lr * grad_scale, 0, m->side);
            // push my shard of the new weights to every peer
            const char* mine = static_cast<const char*>(m->peer[m->rank]) + m->w_off[l] + shard_byte0;
            for (int k = 1; k < m->world; k++) {
                const int p = (m->rank + k) % m->world;
                cudaMemcpyAsync(static_cast<char*>(m->peer[p]) + m->w_off[l] + shard_byte0, mine, shard_bytes, cudaMemcpyDeviceToDevice, m->side);
            }
        } else {
            mx_dp_reduce_sgd(m->is_bf16 ? 0 : 1, m->peer, m->mc, nullptr, m->rank, m->world, m->gw_off[l], m->w_off[l], m->gb_off[l], m->w32[l],
                             m->shard_begin, m->shard_elems, m->b32[l], m->b16[l], lr * grad_scale, m->mc ? m->exclusive_sms : 0, m->side);
        }
        mx_dp_barrier(m->peer, flag_off, m->rank, m->world, ++m->epoch, m->dp_err, m->side);
        cudaEventRecord(m->ev_done[l], m->side);
    };
    auto input_part = [&](int l) {
        if (m->is_bf16) backward_input_t<bf16>(m, l);
        else backward_input_t<f16>(m, l);
    };
    auto weight_part = [&](int l) {
        if (m->is_bf16) backward_weight_t<bf16>(m, l);
        else backward_weight_t<f16>(m, l);
    };
    // Layers L-1 .. 2 in the natural order.  The last two are finished in the order 0, 1: the next forward
    // needs W[0] first, so its exchange starts one GEMM earlier and runs beside dW[1], and the exchange of
    // layer 1 - now the last - runs beside the next step's first layer instead of in front of it.
    for (int l = m->layers - 1; l >= 2; l--) {
        input_part(l);
        weight_part(l);
        exchange(l);
    }
    if (m->layers >= 2) {
        input_part(1);
        input_part(0);
        weight_part(0);
        exchange(0);
        weight_part(1);
        exchange(1);
    } else {
        input_part(0);
        weight_part(0);
        exchange(0);
    }
    ctx().gemm_sm_limit = saved_limit;
    check_launch("mx_mlp_train_step_dp");
}

// How mx_mlp_train_step_dp moves the data: 0 = the library's kernel over NVLink (multimem when the engine
// has a multicast address, peer loads and stores otherwise; exclusive_sms = k > 0 gives the multimem form k SMs
// of its own and the step's GEMMs the rest), 1 = copy engines for the transfers and a local kernel for the sum
// and the update.  Returns 0, or -1 when the staging buffers cannot be allocated.
int mx_mlp_dp_set_exchange(void* h, int mode, int exclusive_sms) {
    Mlp* m = static_cast<Mlp*>(h);
    if (!m->dp || (mode != 0 && mode != 1) || exclusive_sms < 0) return -1;
    m->exclusive_sms = mode == 0 ? exclusive_sms : 0;
    if (mode == 1) {
        for (int p = 0; p < m->world; p++) {
            if (p == m->rank || m->staging[p]) continue;
            m->staging[p] = dmalloc(m, m->shard_elems * 2);
            if (!m->staging[p]) return -1;
        }
    }
    m->copy_engines = mode == 1;
    return 0;
}

// The calling thread's stream waits (on the device) for the exchange of the last step.
// Also valid for the single-device engine after mx_mlp_train_step (its updates run on the side stream).
void mx_mlp_dp_join(void* h) {
    Mlp* m = static_cast<Mlp*>(h);
    for (int l = 0; l < m->layers && l < (int)m->ev_done.size(); l++) cudaStreamWaitEvent(ctx().stream, m->ev_done[l], 0);
}

// Waits for the exchange of the last step and returns 0, or 1 + the peer rank a barrier stopped waiting for.
uint32_t mx_mlp_dp_status(void* h) {
    Mlp* m = static_cast<Mlp*>(h);
    uint32_t v = 0;
    if (!m->dp) return 0;
    cudaStreamSynchronize(m->side);
    cudaMemcpy(&v, m->dp_err, sizeof(v), cudaMemcpyDeviceToHost);
    return v;
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
