// Data-parallel gradient exchange fused with the optimizer step, over NVLink / NVSwitch.
//
// The reference trains on one device; its SGD step is `param.sub_(grad.mul_scalar(lr))`
// (crates/maidenx_nn/src/optimizers/sgd.rs:17-26).  Data-parallel ranks must apply the SUM of all
// ranks' gradients.  The library route is an all-reduce of every gradient (each rank receives the
// full sum) followed by a full-size update on every rank.  Here the two are one kernel per layer
// and each rank touches only 1/world of the parameters:
//
//   rank r, for its shard [r * n / world, (r + 1) * n / world) of a layer's weights:
//     g   = sum over ranks of grad[shard]      multimem.ld_reduce: NVSwitch adds the ranks' copies
//                                              in f32 and returns one 16-byte vector
//                                              (or, without multicast: one peer load per rank)
//     w32 = w32 - lr * scale * g               f32 master copy, kept only for the shard
//     W[shard] on EVERY rank = round(w32)      multimem.st: one store, the switch writes all copies
//                                              (or one peer store per rank)
//
// Per layer and GPU, n * 2 bytes leave and n * 2 bytes enter over NVLink (an all-reduce moves
// about 1.75x that at 8 ranks), the update reads and writes 1/world of the master weights instead
// of all of them, and all ranks end up with bit-identical weights by construction.
//
// Buffers.  Every rank owns an "arena" of the same layout, mapped into every other rank (peer
// pointers) and, when available, bound to a multicast address: [flags | per layer: weight
// gradient, 16-bit weights, bias-gradient slot].  The host side allocates and exchanges it
// (symmetric memory of torch.distributed, or any other allocator of peer-mapped memory) and hands
// the pointers over; nothing here allocates.
//
// Ordering.  dp_barrier_kernel is a flag barrier across ranks: one thread per peer stores the
// epoch into its slot of that peer's flags (release, system scope) and waits for the peer's
// epoch in the local flags (acquire), for at most kWaitCycles; a wait that runs out records
// 1 + peer in the error word and returns, so a lost rank costs seconds, not a hung GPU.
// One barrier before the exchange (every rank's gradient of the layer is complete, and nobody
// still reads the old weights) and one after it (every shard of the new weights has landed).
// The waiting kernels run on different GPUs, one per GPU, so they are always co-resident.
#include <cstdlib>
#include <mutex>

#include "abi_common.cuh"
#include "ops.cuh"

namespace mx {

constexpr int kDpMaxWorld = 16;
constexpr long long kWaitCycles = 4000000000ll;  // about two seconds of SM clock

struct DpPeers {
    void* base[kDpMaxWorld];  // arena of rank p as mapped into this process; base[rank] is the local one
};

__global__ void dp_barrier_kernel(DpPeers peers, size_t flag_off, int rank, int world, uint32_t epoch, uint32_t* err) {
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();  // everything this GPU wrote before the barrier is visible before the flag
    uint32_t* theirs = reinterpret_cast<uint32_t*>(static_cast<char*>(peers.base[p]) + flag_off) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(static_cast<char*>(peers.base[rank]) + flag_off) + p;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;  // epochs only grow; a peer may already be one barrier ahead
        if (clock64() - t0 > kWaitCycles) {
            atomicCAS(err, 0u, 1u + (uint32_t)p);
            break;
        }
        __nanosleep(200);
    }
}

template <class T>
__device__ __forceinline__ uint4 multimem_ld_reduce(const void* mc_addr);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<bf16>(const void* mc_addr) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc_addr)
                 : "memory");
    return r;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<f16>(const void* mc_addr) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc_addr)
                 : "memory");
    return r;
}
template <class T>
__device__ __forceinline__ void multimem_st(void* mc_addr, uint4 v);
template <>
__device__ __forceinline__ void multimem_st<bf16>(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <>
__device__ __forceinline__ void multimem_st<f16>(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

constexpr int kDpThreads = 256;
constexpr int kDpMaxThreads = 1024;
// A CTA that asks for this much shared memory cannot share an SM with a CTA of the tensor-core GEMM (about
// 200 KB), nor with a second one of its own kind: with the GEMM launched on sm_count - k CTAs, k such CTAs get k
// SMs to themselves and the GEMM's own waits are never queued behind NVLink round trips.
constexpr int kDpExclusiveSmem = 120 * 1024;
constexpr int kDpUnroll = 4;  // 16-byte vectors in flight per thread: NVLink round trips are several microseconds

struct DpLayer {
    size_t grad_off, weight_off, bias_grad_off;  // byte offsets inside every arena
    float* master_shard;                         // f32 master weights of this rank's shard
    size_t shard_begin, shard_elems;             // in elements; both multiples of 8
    float* master_bias;                          // f32 master bias (every rank keeps the scalar)
    void* bias16;                                // local 16-bit working copy of the bias
    const void* staged[kDpMaxWorld];             // kStaged: local copies of the peers' gradient shards ([rank] unused)
};

enum { kMulticast = 0, kPeer = 1, kStaged = 2 };

// MODE kMulticast: sums and broadcasts go through the multicast address.
// MODE kPeer: one peer load and one peer store per rank.
// MODE kStaged: the peers' shards were copied into local memory beforehand (copy engines) and the new
// weights are written to the local arena only (the host pushes them to the peers afterwards); the SMs
// then never wait on NVLink.
// In the last two, ranks are added in rank order, so every run and every rank rounds the same way.
template <class T, int MODE>
__global__ void __launch_bounds__(MODE == kMulticast ? kDpMaxThreads : kDpThreads) dp_reduce_sgd_kernel(DpPeers peers, char* mc_base, DpLayer L, int rank, int world, float step, int) {
    constexpr int UNROLL = MODE == kMulticast ? kDpUnroll : 2;
    const size_t nvec = L.shard_elems / 8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * UNROLL) {
        uint4 g[UNROLL];
        if constexpr (MODE == kMulticast) {
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const size_t v = v0 + u * stride;
                if (v < nvec) g[u] = multimem_ld_reduce<T>(mc_base + L.grad_off + (L.shard_begin + v * 8) * 2);
            }
        } else {
            // all loads of the trip first (up to 8 ranks x UNROLL vectors in flight), then the sums
            constexpr int W = 8;
            for (int p0 = 0; p0 < world; p0 += W) {
                uint4 x[UNROLL][W];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    const size_t v = v0 + u * stride;
#pragma unroll
                    for (int q = 0; q < W; q++) {
                        const int p = p0 + q;
                        if (p < world && v < nvec) {
                            const char* src = (MODE == kStaged && p != rank) ? static_cast<const char*>(L.staged[p]) + v * 16
                                                                            : static_cast<const char*>(peers.base[p]) + L.grad_off + (L.shard_begin + v * 8) * 2;
                            x[u][q] = __ldcv(reinterpret_cast<const uint4*>(src));
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    float acc[8];
                    if (p0 == 0) {
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[j] = 0.0f;
                    } else {  // more than 8 ranks: continue from the running sum (kept as f32 bit patterns would cost registers; re-expand)
                        const uint32_t w[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float2 f = unpack2<T>(w[j]);
                            acc[2 * j] = f.x;
                            acc[2 * j + 1] = f.y;
                        }
                    }
#pragma unroll
                    for (int q = 0; q < W; q++) {
                        if (p0 + q < world) {
                            const uint32_t w[4] = {x[u][q].x, x[u][q].y, x[u][q].z, x[u][q].w};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const float2 f = unpack2<T>(w[j]);
                                acc[2 * j] += f.x;
                                acc[2 * j + 1] += f.y;
                            }
                        }
                    }
                    g[u] = make_uint4(pack2_rn<T>(acc[0], acc[1]), pack2_rn<T>(acc[2], acc[3]), pack2_rn<T>(acc[4], acc[5]), pack2_rn<T>(acc[6], acc[7]));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const size_t v = v0 + u * stride;
            if (v >= nvec) break;
            float4* m = reinterpret_cast<float4*>(L.master_shard + v * 8);
            float4 m0 = m[0], m1 = m[1];
            const uint32_t w[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
            float gf[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = unpack2<T>(w[j]);
                gf[2 * j] = f.x;
                gf[2 * j + 1] = f.y;
            }
            m0.x = m0.x - step * gf[0];
            m0.y = m0.y - step * gf[1];
            m0.z = m0.z - step * gf[2];
            m0.w = m0.w - step * gf[3];
            m1.x = m1.x - step * gf[4];
            m1.y = m1.y - step * gf[5];
            m1.z = m1.z - step * gf[6];
            m1.w = m1.w - step * gf[7];
            m[0] = m0;
            m[1] = m1;
            const uint4 out = make_uint4(pack2_rn<T>(m0.x, m0.y), pack2_rn<T>(m0.z, m0.w), pack2_rn<T>(m1.x, m1.y), pack2_rn<T>(m1.z, m1.w));
            const size_t byte = L.weight_off + (L.shard_begin + v * 8) * 2;
            if constexpr (MODE == kMulticast) {
                multimem_st<T>(mc_base + byte, out);
            } else if constexpr (MODE == kPeer) {
                for (int p = 0; p < world; p++) __stwt(reinterpret_cast<uint4*>(static_cast<char*>(peers.base[p]) + byte), out);
            } else {
                *reinterpret_cast<uint4*>(static_cast<char*>(peers.base[rank]) + byte) = out;
            }
        }
    }
    // the scalar bias: every rank adds the ranks' gradients in rank order and updates its own copy
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        float acc = 0.0f;
        for (int p = 0; p < world; p++) {
            const unsigned short bits = __ldcv(reinterpret_cast<const unsigned short*>(static_cast<const char*>(peers.base[p]) + L.bias_grad_off));
            acc += to_f32(*reinterpret_cast<const T*>(&bits));
        }
        const float gsum = to_f32(from_f32<T>(acc));  // the sum a 16-bit all-reduce would deliver
        const float b = *L.master_bias - step * gsum;
        *L.master_bias = b;
        *static_cast<T*>(L.bias16) = from_f32<T>(b);
    }
    __threadfence_system();  // the broadcast stores are performed before this rank reports "done"
}

template <class T>
static void dp_reduce_sgd_launch(const DpPeers& peers, void* mc_base, const DpLayer& L, bool staged, int exclusive_sms, int rank, int world, float step,
                                 cudaStream_t s, const char* where) {
    if (world < 1 || world > kDpMaxWorld || rank < 0 || rank >= world || L.shard_elems % 8 || L.shard_begin % 8) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    const size_t nvec = L.shard_elems / 8;
    if (exclusive_sms > 0 && !staged && mc_base) {
        // k CTAs of 1024 threads, one per SM, kept apart from the GEMM by their shared-memory request
        // the opt-in to large dynamic shared memory is a per-device function attribute
        static std::mutex mu;
        static bool opted_in[64] = {false};
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
            set_error(kErrNoDevice, 0, where);
            return;
        }
        {
            std::lock_guard<std::mutex> lock(mu);
            if (!opted_in[dev]) {
                if (cudaFuncSetAttribute(dp_reduce_sgd_kernel<T, kMulticast>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDpExclusiveSmem) != cudaSuccess) {
                    set_error(kErrCuda, (int)cudaGetLastError(), where);
                    return;
                }
                opted_in[dev] = true;
            }
        }
        dp_reduce_sgd_kernel<T, kMulticast><<<exclusive_sms, kDpMaxThreads, kDpExclusiveSmem, s>>>(peers, static_cast<char*>(mc_base), L, rank, world, step, 0);
        check_launch(where);
        return;
    }
    size_t blocks = (nvec + (size_t)kDpThreads * 2 - 1) / ((size_t)kDpThreads * 2);
    size_t cap = (size_t)sm_count() * 2;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (staged) dp_reduce_sgd_kernel<T, kStaged><<<(unsigned)blocks, kDpThreads, 0, s>>>(peers, nullptr, L, rank, world, step, 0);
    else if (mc_base) dp_reduce_sgd_kernel<T, kMulticast><<<(unsigned)blocks, kDpThreads, 0, s>>>(peers, static_cast<char*>(mc_base), L, rank, world, step, 0);
    else dp_reduce_sgd_kernel<T, kPeer><<<(unsigned)blocks, kDpThreads, 0, s>>>(peers, nullptr, L, rank, world, step, 0);
    check_launch(where);
}

}  // namespace mx

using namespace mx;

extern "C" {

// One flag barrier across `world` ranks on `stream` (a cudaStream_t; NULL = the calling thread's
// current stream).  peer_arenas[p] + flag_offset is an array of `world` u32 flags in rank p's arena,
// zero before the first barrier; `epoch` must grow by one per barrier.  err: device word, 0 = fine.
void mx_dp_barrier(void* const* peer_arenas, size_t flag_offset, int rank, int world, uint32_t epoch, uint32_t* err, void* stream) {
    if (world < 1 || world > kDpMaxWorld || rank < 0 || rank >= world) {
        set_error(kErrBadMetadata, 0, "mx_dp_barrier");
        return;
    }
    DpPeers peers;
    for (int p = 0; p < kDpMaxWorld; p++) peers.base[p] = p < world ? peer_arenas[p] : nullptr;
    cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : ctx().stream;
    dp_barrier_kernel<<<1, 32, 0, s>>>(peers, flag_offset, rank, world, epoch, err);
    check_launch("mx_dp_barrier");
}

// The fused exchange + SGD step of one layer for this rank's shard (see the top of this file).
// dtype: 0 = bf16, 1 = f16.  multicast_arena: the arenas' multicast address, or NULL to use peer
// loads and stores.  staged_grads: NULL, or `world` pointers to local copies of the ranks' gradient
// shards (entry [rank] is ignored: the own shard is read in place); then the new weights are written
// to the local arena only and the caller copies them to the peers.  step = lr * grad_scale.  Offsets
// are bytes inside every arena.  exclusive_sms: 0 = blocks spread over all SMs; k > 0 = k blocks of 1024
// threads that keep an SM each to themselves (multicast form only; see kDpExclusiveSmem; pair it with
// mx_set_gemm_sm_limit).
void mx_dp_reduce_sgd(int dtype, void* const* peer_arenas, void* multicast_arena, const void* const* staged_grads, int rank, int world,
                      size_t grad_offset, size_t weight_offset, size_t bias_grad_offset, float* master_shard, size_t shard_begin, size_t shard_elems,
                      float* master_bias, void* bias16, float step, int exclusive_sms, void* stream) {
    DpPeers peers;
    for (int p = 0; p < kDpMaxWorld; p++) peers.base[p] = (p < world && world <= kDpMaxWorld) ? peer_arenas[p] : nullptr;
    DpLayer L;
    L.grad_off = grad_offset;
    L.weight_off = weight_offset;
    L.bias_grad_off = bias_grad_offset;
    L.master_shard = master_shard;
    L.shard_begin = shard_begin;
    L.shard_elems = shard_elems;
    L.master_bias = master_bias;
    L.bias16 = bias16;
    for (int p = 0; p < kDpMaxWorld; p++) L.staged[p] = (staged_grads && p < world && world <= kDpMaxWorld) ? staged_grads[p] : nullptr;
    const bool staged = staged_grads != nullptr;
    cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : ctx().stream;
    if (dtype == 0) dp_reduce_sgd_launch<bf16>(peers, multicast_arena, L, staged, exclusive_sms, rank, world, step, s, "mx_dp_reduce_sgd");
    else if (dtype == 1) dp_reduce_sgd_launch<f16>(peers, multicast_arena, L, staged, exclusive_sms, rank, world, step, s, "mx_dp_reduce_sgd");
    else set_error(kErrUnsupported, 0, "mx_dp_reduce_sgd");
}

}  // extern "C"
