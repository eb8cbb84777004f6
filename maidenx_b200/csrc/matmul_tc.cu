// Tensor-core path for bf16 / f16 matmul on sm_100a: tcgen05.mma with the accumulator in
// tensor memory (TMEM), operands staged in shared memory by TMA, epilogue read back with
// tcgen05.ld, converted and written with TMA stores.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the A [128 x 64]
//               and B [256 x 64] k-blocks into a 4-stage shared-memory ring (128-byte swizzle);
//   warp 1      MMA issuer: one lane issues four tcgen05.mma (M128 N256 K16) per k-block into
//               one of two 256-column TMEM accumulators, commits the stage back to the
//               producer and, after the last k-block, the accumulator to the epilogue;
//   warps 2-5   epilogue: each warp owns the 32 TMEM lanes it may address (warp id mod 4),
//               reads them 64 columns at a time, rounds to bf16 / f16, writes a swizzled
//               4 KB staging tile and stores it with TMA while the next tile's MMAs run on
//               the other accumulator.
// No cluster launch: every CTA issues its own (CTA-local) TMA loads; re-use comes from
// L2 through the order in which output tiles are handed out (16 row-tiles per column sweep).
//
// The kernel computes D[M,N] = sum_k A[m,k] * B[n,k]; by default both operands are K-major (row-major
// [M,K] and [N,K]): the reference's forward x . W^T (crates/maidenx_nn/src/layers/linear.rs:74) and
// its grad_a = g . B^T (crates/maidenx_cpu/src/ops/matmul.rs:208-216).  Either operand may instead be
// MN-major (row-major [K,M] / [K,N]): it is then loaded as 64-wide column chunks and described
// to the tensor core with the MN-major descriptor form, which covers grad_b = A^T . g (:244-256)
// and a plain [K,N] B without any transposed copy.
//
// Every mbarrier wait is bounded by a clock64() budget; on expiry the thread records an
// error word, stops issuing work and falls through to the common exit, where TMEM is freed.
#include <cuda.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "matmul_tc.cuh"
#include "matmul_tc2.cuh"
#include "tc_ptx.cuh"

namespace mx {

using namespace tc;

namespace {

// true: products go to the two-CTA kernel (matmul_tc2.cu); false (default): to the one-CTA kernel below.  On a B200 under
// its power cap the two run at the same rate (the pair form only moves less data through shared memory).
std::atomic<bool> g_two_cta{false};
std::atomic<int> g_group_m{16};  // row-tiles per column sweep of the one-CTA kernel's tile order

constexpr int BM = 128, BN = 256, BK = 64;    // CTA tile; BK * 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;    // 32 KB
constexpr int EPI_WARPS = 4;
constexpr int EPI_CHUNK_COLS = 64;            // columns per TMA store (128 bytes of 16-bit)
constexpr int EPI_STAGE_BYTES = 32 * EPI_CHUNK_COLS * 2;  // 4 KB per warp per buffer
constexpr int TC_THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = 512;                // two 256-column f32 accumulators
constexpr int GROUP_M = 16;                   // row-tiles per column sweep (L2 re-use)

struct SmemLayout {
    // offsets inside the dynamic shared memory block (base aligned to 1024 bytes)
    static constexpr int a = 0;
    static constexpr int b = a + STAGES * A_STAGE_BYTES;
    static constexpr int epi = b + STAGES * B_STAGE_BYTES;
    static constexpr int bars = epi + EPI_WARPS * 2 * EPI_STAGE_BYTES;
    static constexpr int total = bars + 256;
};
constexpr int TC_SMEM_BYTES = SmemLayout::total + 1024;  // slack for the 1024-byte alignment

constexpr int MN_CHUNK_BYTES = 64 * BK * 2;  // one [64 K-rows x 64 MN] box

// Instruction descriptor of tcgen05.mma kind::f16 with f32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc(bool is_bf16, bool a_mn_major, bool b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;                               // D format: f32
    d |= (is_bf16 ? 1u : 0u) << 7;              // A format: 0 = f16, 1 = bf16
    d |= (is_bf16 ? 1u : 0u) << 10;             // B format
    d |= (a_mn_major ? 1u : 0u) << 15;          // A major: 0 = K, 1 = MN
    d |= (b_mn_major ? 1u : 0u) << 16;          // B major
    d |= (uint32_t)(BN >> 3) << 17;             // N / 8
    d |= (uint32_t)(BM >> 4) << 24;             // M / 16
    return d;
}

struct TcParams {
    int M, N, K;
    int tiles_m, tiles_n, num_tiles, num_kb;
    int tiles_per_batch;   // tiles_m * tiles_n; num_tiles = batch * tiles_per_batch
    int a_batched, b_batched;  // 0: the operand is one matrix shared by every batch (third TMA coordinate stays 0)
    int is_bf16;
    int out_f32;  // split-K partial results: the epilogue stores the f32 accumulators unrounded
    int fuse;     // 0: store the product; 1: u = round(round(product) + bias) through map_d; 2: also act = round(gelu(u)) through map_d2;
                  // 3: as 1 with one bias element per output ROW (bias[row of the batch's matrix]): a convolution's per-channel bias
    const void* bias;  // fuse != 0: one element of the operand type in device memory
    int a_mn, b_mn;  // operand is MN-major in global memory ([K, MN] row-major) instead of K-major ([MN, K])
    int group_m;     // row-tiles per column sweep (L2 re-use of the A panels)
    // Short reductions (num_kb <= STAGES, one batch): `b_keep` CTAs share each column tile, CTA j of them takes the row
    // tiles j, j + b_keep, ...; the B panel of the column tile is loaded once into the B slots of the ring (slot = k-block,
    // the ring is num_kb slots long) and only A streams.  0: the general schedule.
    int b_keep;
};

__device__ __forceinline__ void tile_coords(int tile, const TcParams& p, int& tm, int& tn, int& tb) {
    tb = tile / p.tiles_per_batch;
    tile -= tb * p.tiles_per_batch;
    // sweep GROUP_M row-tiles for each column tile before moving to the next column tile
    const int group_size = p.group_m * p.tiles_n;
    const int group = tile / group_size;
    const int first_m = group * p.group_m;
    const int rows = min(p.group_m, p.tiles_m - first_m);
    const int in_group = tile - group * group_size;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

// The it-th tile of this CTA; false when it has none left.
__device__ __forceinline__ bool next_tile(int it, const TcParams& p, int& tm, int& tn, int& tb) {
    if (p.b_keep) {
        tn = (int)blockIdx.x / p.b_keep;
        tm = (int)blockIdx.x % p.b_keep + it * p.b_keep;
        tb = 0;
        return tn < p.tiles_n && tm < p.tiles_m;
    }
    const int tile = (int)blockIdx.x + it * (int)gridDim.x;
    if (tile >= p.num_tiles) return false;
    tile_coords(tile, p, tm, tn, tb);
    return true;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// v rounded to the operand type and widened again
__device__ __forceinline__ float round16(float v, int is_bf16) {
    return is_bf16 ? to_f32(from_f32<bf16>(v)) : to_f32(from_f32<f16>(v));
}

__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_d,
               const __grid_constant__ CUtensorMap map_d2, TcParams p, int* err, int tag) {
    extern __shared__ unsigned char tc_smem_raw[];
    // 128-byte swizzled TMA tiles and UMMA descriptors want 1024-byte aligned bases
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + SmemLayout::bars;
    // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM base word
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + SmemLayout::bars + 8 * (2 * STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), EPI_WARPS);
        }
        fence_barrier_init();
    }
    if (warp == 1) {  // the MMA warp owns the TMEM allocation
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int ring = p.b_keep ? p.num_kb : STAGES;
            int tm, tn, tb;
            for (int it = 0; ok && next_tile(it, p, tm, tn, tb); it++) {
                const int za = p.a_batched ? tb : 0, zb = p.b_batched ? tb : 0;
                const bool load_b = !p.b_keep || it == 0;  // the kept B panel arrives with the first tile's A blocks
                for (int kb = 0; kb < p.num_kb; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, err, tag, 1)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full_bar(stage), A_STAGE_BYTES + (load_b ? B_STAGE_BYTES : 0));
                    const uint32_t sa = smem_base + SmemLayout::a + stage * A_STAGE_BYTES;
                    const uint32_t sb = smem_base + SmemLayout::b + stage * B_STAGE_BYTES;
                    if (!p.a_mn) {
                        tma_load_3d(sa, &map_a, kb * BK, tm * BM, za, full_bar(stage));
                    } else {
#pragma unroll
                        for (int h = 0; h < BM / 64; h++) tma_load_3d(sa + h * MN_CHUNK_BYTES, &map_a, tm * BM + h * 64, kb * BK, za, full_bar(stage));
                    }
                    if (!load_b) {
                    } else if (!p.b_mn) {
                        tma_load_3d(sb, &map_b, kb * BK, tn * BN, zb, full_bar(stage));
                    } else {
#pragma unroll
                        for (int h = 0; h < BN / 64; h++) tma_load_3d(sb + h * MN_CHUNK_BYTES, &map_b, tn * BN + h * 64, kb * BK, zb, full_bar(stage));
                    }
                    if (++stage == ring) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(p.is_bf16 != 0, p.a_mn != 0, p.b_mn != 0);
            // per-operand descriptor geometry: (leading, stride) byte offsets and the K step in 16-byte units
            const uint32_t a_lbo = p.a_mn ? MN_CHUNK_BYTES : 16, b_lbo = p.b_mn ? MN_CHUNK_BYTES : 16;
            const uint64_t a_kstep = p.a_mn ? (2048 >> 4) : (32 >> 4), b_kstep = p.b_mn ? (2048 >> 4) : (32 >> 4);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const int ring = p.b_keep ? p.num_kb : STAGES;
            int tm, tn, tb;
            for (int it = 0; ok && next_tile(it, p, tm, tn, tb); it++) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, err, tag, 2)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
                for (int kb = 0; kb < p.num_kb; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, err, tag, 3)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = smem_desc_sw128(smem_base + SmemLayout::a + stage * A_STAGE_BYTES, a_lbo, 1024);
                    const uint64_t db = smem_desc_sw128(smem_base + SmemLayout::b + stage * B_STAGE_BYTES, b_lbo, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) umma_f16(d_tmem, da + a_kstep * k, db + b_kstep * k, idesc, (kb | k) != 0);
                    umma_commit(empty_bar(stage));  // the stage may be refilled once these MMAs have read it
                    if (++stage == ring) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(tfull_bar(acc));  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;  // TMEM lanes [32 * quarter, 32 * quarter + 32)
        const int ew = warp - 2;
        unsigned char* stage_buf = smem + SmemLayout::epi + ew * 2 * EPI_STAGE_BYTES;
        int acc = 0, buf = 0;
        uint32_t acc_phase = 0;
        float fused_bias = 0.0f;
        if (p.fuse == 1 || p.fuse == 2) fused_bias = p.is_bf16 ? to_f32(*static_cast<const bf16*>(p.bias)) : to_f32(*static_cast<const f16*>(p.bias));
        int tm, tn, tb;
        for (int it = 0; next_tile(it, p, tm, tn, tb); it++) {
            // the TMEM loads below are warp-collective: leave the loop only as a whole warp
            // four warps wait here for most of a tile's reduction: they sleep between polls, so that their polling does not
            // take shared-memory cycles from the TMA writes and the tensor core's operand reads
            if (p.fuse == 3) {  // this thread's output row inside the batch's matrix
                const int row = tm * BM + quarter * 32 + lane;
                fused_bias = row < p.M ? (p.is_bf16 ? to_f32(static_cast<const bf16*>(p.bias)[row]) : to_f32(static_cast<const f16*>(p.bias)[row])) : 0.0f;
            }
            const bool ready = mbar_wait_relaxed(tfull_bar(acc), acc_phase, err, tag, 4, 400);
            if (!__all_sync(0xFFFFFFFFu, ready)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
            // One 64-column chunk: round, stage in shared memory (XOR-swizzled rows), hand to the copy engine.
            auto store_chunk = [&](int c, uint32_t (&v0)[32], uint32_t (&v1)[32]) {
                if (p.fuse) {
                    // Linear + bias (+ GELU) in one pass, with the roundings of the separate ops: the product is rounded to
                    // the operand type, the bias is added in f32 and rounded (u), the activation is evaluated on u in f32
                    // and rounded (act) - bit for bit what cuda_matmul, cuda_add and cuda_gelu give one after the other.
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        v0[j] = __float_as_uint(round16(round16(__uint_as_float(v0[j]), p.is_bf16) + fused_bias, p.is_bf16));
                        v1[j] = __float_as_uint(round16(round16(__uint_as_float(v1[j]), p.is_bf16) + fused_bias, p.is_bf16));
                    }
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        if (h == 1 && p.fuse != 2) break;
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                        unsigned char* dst = stage_buf + buf * EPI_STAGE_BYTES + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const uint32_t* src = j < 4 ? &v0[j * 8] : &v1[(j - 4) * 8];
                            float e[8];
#pragma unroll
                            for (int k = 0; k < 8; k++) e[k] = h ? gelu_f32_fast(__uint_as_float(src[k])) : __uint_as_float(src[k]);  // second pass: the activation of u
                            uint4 q;
                            q.x = pack2(e[0], e[1], p.is_bf16);
                            q.y = pack2(e[2], e[3], p.is_bf16);
                            q.z = pack2(e[4], e[5], p.is_bf16);
                            q.w = pack2(e[6], e[7], p.is_bf16);
                            *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = q;
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(h ? &map_d2 : &map_d, smem_u32(stage_buf + buf * EPI_STAGE_BYTES), tn * BN + c * EPI_CHUNK_COLS, tm * BM + quarter * 32, tb);
                            tma_store_commit();
                        }
                        buf ^= 1;
                    }
                    return;
                }
                if (p.out_f32) {
                    // two 32-column f32 chunks (128 bytes per row each), one per staging buffer
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t* v = h ? v1 : v0;
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                        unsigned char* dst = stage_buf + buf * EPI_STAGE_BYTES + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&map_d, smem_u32(stage_buf + buf * EPI_STAGE_BYTES), tn * BN + c * EPI_CHUNK_COLS + h * 32, tm * BM + quarter * 32, tb);
                            tma_store_commit();
                        }
                        buf ^= 1;
                    }
                    return;
                }
                // the staging buffer must have been read by its previous TMA store
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                unsigned char* dst = stage_buf + buf * EPI_STAGE_BYTES + lane * 128;  // row `lane` of the 32 x 64 tile
#pragma unroll
                for (int j = 0; j < 8; j++) {  // eight 16-byte chunks per row, XOR-swizzled by the row index
                    const uint32_t* src = j < 4 ? &v0[j * 8] : &v1[(j - 4) * 8];
                    uint4 q;
                    q.x = pack2(__uint_as_float(src[0]), __uint_as_float(src[1]), p.is_bf16);
                    q.y = pack2(__uint_as_float(src[2]), __uint_as_float(src[3]), p.is_bf16);
                    q.z = pack2(__uint_as_float(src[4]), __uint_as_float(src[5]), p.is_bf16);
                    q.w = pack2(__uint_as_float(src[6]), __uint_as_float(src[7]), p.is_bf16);
                    *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = q;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&map_d, smem_u32(stage_buf + buf * EPI_STAGE_BYTES), tn * BN + c * EPI_CHUNK_COLS, tm * BM + quarter * 32, tb);
                    tma_store_commit();
                }
                buf ^= 1;
            };
            // The TMEM loads of chunk c + 1 are in flight while chunk c is converted and stored.
            uint32_t a0[32], a1[32], b0[32], b1[32];
            tmem_ld_32x32b_x32(t_row, a0);
            tmem_ld_32x32b_x32(t_row + 32, a1);
#pragma unroll
            for (int c = 0; c < BN / EPI_CHUNK_COLS; c += 2) {
                tmem_ld_wait_for(a0);
                reg_fence(a1);
                tmem_ld_32x32b_x32(t_row + (c + 1) * EPI_CHUNK_COLS, b0);
                tmem_ld_32x32b_x32(t_row + (c + 1) * EPI_CHUNK_COLS + 32, b1);
                store_chunk(c, a0, a1);
                tmem_ld_wait_for(b0);
                reg_fence(b1);
                if (c + 2 < BN / EPI_CHUNK_COLS) {
                    tmem_ld_32x32b_x32(t_row + (c + 2) * EPI_CHUNK_COLS, a0);
                    tmem_ld_32x32b_x32(t_row + (c + 2) * EPI_CHUNK_COLS + 32, a1);
                } else {
                    // every TMEM read of this accumulator is done: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(acc));
                }
                store_chunk(c + 1, b0, b1);
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    // common exit: TMEM is released by the warp that allocated it, after everyone is done with it
    tc_fence_before();
    __syncthreads();
    if (tc_err_mine(err, tag)) {
        // a wait gave up: give bulk copies still in flight towards this CTA's shared memory time to land
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000ll) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
// [rows, cols] row-major 16-bit matrix, box = box_rows x 64 columns, 128-byte swizzle
bool make_map(CUtensorMap* map, bool is_bf16, const void* base, uint64_t rows, uint64_t cols, uint64_t batch, uint64_t batch_stride, uint32_t box_rows) {
    return make_map_3d(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, rows, cols, batch, batch_stride, box_rows);
}

bool opt_in_shared_memory() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
        if (cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        done[dev] = true;
    }
    return true;
}

// D[M,N] = sum_k Aop[m,k] * Bop[n,k].  A K-major operand is a dense row-major [MN, K] matrix, an
// MN-major operand a dense row-major [K, MN] matrix; D is dense row-major [M, N].
// fuse: 0 plain product; 1 D = round(round(product) + bias); 2 also D2 = round(gelu(D)) (see the kernel's epilogue)
std::atomic<int> g_keep_b{1};  // 0: the B-panel-resident schedule is never taken (tests, A/B timing)

// CTAs per column tile of the schedule that keeps the B panel of a column tile in shared memory (0 = general schedule).
// Taken when the whole reduction fits the ring (K <= STAGES * BK), there is one batch, and every CTA gets at least four
// row tiles to spread the panel's load over.  With K = 256 a 128 x 256 tile otherwise loads 192 KB to do 2048 cycles
// of tensor work; with the panel resident it loads the 64 KB of A.
int keep_b_ctas(int tiles_m, int tiles_n, int num_kb, int batch, int ctas) {
    if (!g_keep_b.load(std::memory_order_relaxed) || batch != 1 || num_kb > STAGES || tiles_n > ctas) return 0;
    const int per_col = ctas / tiles_n;
    return tiles_m >= 4 * per_col ? per_col : 0;
}

bool launch_gemm(bool is_bf16, const TcProduct& c, void* D, const char* where, int fuse = 0, const void* bias = nullptr, void* D2 = nullptr) {
    const void *A = c.A, *B = c.B;
    const bool a_mn = c.a_mn, b_mn = c.b_mn;
    const uint64_t M = c.m, N = c.n;
    uint64_t K = c.k, batch = c.batch;
    if (!opt_in_shared_memory()) return false;
    TcParams p;
    p.M = (int)M;
    p.N = (int)N;
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + BN - 1) / BN);
    p.tiles_per_batch = p.tiles_m * p.tiles_n;
    int grid = sm_count();
    if (ctx().gemm_sm_limit > 0 && ctx().gemm_sm_limit < grid) grid = ctx().gemm_sm_limit;
    // few output tiles, long reduction: cut K into slices that run as the batches of this launch
    const int slices = (batch == 1 && !fuse) ? splitk_slices((uint64_t)p.tiles_per_batch, K, BK, grid) : 1;
    float* partial = nullptr;
    uint64_t a_bs = (uint64_t)c.a_bs, b_bs = (uint64_t)c.b_bs, a_pitch = 0, b_pitch = 0;
    if (slices > 1) {
        partial = static_cast<float*>(scratch((size_t)slices * M * N * sizeof(float)));
        if (!partial) return false;
        const uint64_t Ks = K / slices;
        a_pitch = a_mn ? M : K;  // rows keep the pitch of the whole matrix
        b_pitch = b_mn ? N : K;
        a_bs = a_mn ? Ks * M : Ks;  // MN-major: Ks rows further; K-major: Ks columns further
        b_bs = b_mn ? Ks * N : Ks;
        K = Ks;
        batch = (uint64_t)slices;
    }
    int tag = 0;
    int* err = next_launch_error_word(&tag);
    if (!err) return false;
    const CUtensorMapDataType t16 = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
    CUtensorMap ma, mb, md;
    if (g_two_cta.load(std::memory_order_relaxed) && grid >= 2 && !fuse) {
        // the two-CTA kernel: B is staged in halves of 128 columns, a pair of CTAs owns a 256 x 256 tile
        const bool oka2 = a_mn ? make_map_3d(&ma, t16, 2, A, K, M, batch, a_bs, 64, sw, a_pitch) : make_map_3d(&ma, t16, 2, A, M, K, batch, a_bs, tc2::BM, sw, a_pitch);
        const bool okb2 = b_mn ? make_map_3d(&mb, t16, 2, B, K, N, batch, b_bs, 64, sw, b_pitch) : make_map_3d(&mb, t16, 2, B, N, K, batch, b_bs, tc2::BN_HALF, sw, b_pitch);
        const bool okd2 = partial ? make_map_3d(&md, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, partial, M, N, batch, M * N, 32) : make_map(&md, is_bf16, D, M, N, batch, M * N, 32);
        if (oka2 && okb2 && okd2) {
            tc2::Params q;
            q.tile_pairs_m = (p.tiles_m + 1) / 2;
            q.tiles_n = p.tiles_n;
            q.tiles_per_batch = q.tile_pairs_m * q.tiles_n;
            q.num_tiles = (int)batch * q.tiles_per_batch;
            q.num_kb = (int)((K + BK - 1) / BK);
            q.a_batched = (batch > 1 && a_bs != 0) ? 1 : 0;
            q.b_batched = (batch > 1 && b_bs != 0) ? 1 : 0;
            q.is_bf16 = is_bf16 ? 1 : 0;
            q.out_f32 = partial ? 1 : 0;
            q.a_mn = a_mn ? 1 : 0;
            q.b_mn = b_mn ? 1 : 0;
            if (tc2::launch(ma, mb, md, q, grid, err, tag, ctx().stream)) {
                check_launch(where);
                if (partial) splitk_reduce(is_bf16 ? 0 : 1, partial, slices, (size_t)(M * N), D, where);
                return true;
            }
        }
    }
    const bool oka = a_mn ? make_map_3d(&ma, t16, 2, A, K, M, batch, a_bs, 64, sw, a_pitch) : make_map_3d(&ma, t16, 2, A, M, K, batch, a_bs, BM, sw, a_pitch);
    const bool okb = b_mn ? make_map_3d(&mb, t16, 2, B, K, N, batch, b_bs, 64, sw, b_pitch) : make_map_3d(&mb, t16, 2, B, N, K, batch, b_bs, BN, sw, b_pitch);
    const bool okd = partial ? make_map_3d(&md, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, partial, M, N, batch, M * N, 32) : make_map(&md, is_bf16, D, M, N, batch, M * N, 32);
    if (!oka || !okb || !okd) return false;
    CUtensorMap md2 = md;
    if (fuse == 2 && !make_map(&md2, is_bf16, D2, M, N, batch, M * N, 32)) return false;
    p.fuse = fuse;
    p.bias = bias;
    p.group_m = g_group_m.load(std::memory_order_relaxed);
    p.K = (int)K;
    p.num_tiles = (int)batch * p.tiles_per_batch;
    p.a_batched = (batch > 1 && a_bs != 0) ? 1 : 0;
    p.b_batched = (batch > 1 && b_bs != 0) ? 1 : 0;
    p.num_kb = (int)((K + BK - 1) / BK);
    p.is_bf16 = is_bf16 ? 1 : 0;
    p.out_f32 = partial ? 1 : 0;
    p.a_mn = a_mn ? 1 : 0;
    p.b_mn = b_mn ? 1 : 0;
    if (grid > p.num_tiles) grid = p.num_tiles;
    p.b_keep = keep_b_ctas(p.tiles_m, p.tiles_n, p.num_kb, (int)batch, grid);
    if (p.b_keep) grid = p.b_keep * p.tiles_n;
    tc_gemm_kernel<<<grid, TC_THREADS, TC_SMEM_BYTES, ctx().stream>>>(ma, mb, md, md2, p, err, tag);
    check_launch(where);
    if (partial) splitk_reduce(is_bf16 ? 0 : 1, partial, slices, (size_t)(M * N), D, where);
    return true;
}

}  // namespace

// ---------------------------------------------------------------------------------
// shared host helpers (declared in tc_ptx.cuh)
// ---------------------------------------------------------------------------------
namespace tc {

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

bool make_map_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_map_3d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t rows, uint64_t cols, uint64_t batch,
                 uint64_t batch_stride, uint32_t box_rows, CUtensorMapSwizzle swizzle, uint64_t pitch) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    if (pitch == 0) pitch = cols;
    const bool bcast = batch_stride == 0 || batch <= 1;
    cuuint64_t dims[3] = {cols, rows, bcast ? 1 : batch};
    cuuint64_t strides[2] = {pitch * (uint64_t)elem_bytes, (bcast ? rows * pitch : batch_stride) * (uint64_t)elem_bytes};
    cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, type, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

int splitk_slices(uint64_t tiles, uint64_t K, int block_k, int sms) {
    if (tiles == 0 || tiles * 2 > (uint64_t)sms || K % block_k != 0 || K < 4096) return 1;
    const uint64_t kb = K / block_k;
    // Cost in units of one k-block of tensor-core time per CTA: every wave runs kb / s k-blocks plus about 12 for the
    // pipeline fill and the f32 epilogue of a tile, and the second pass reads s partial tiles per output tile.
    auto cost = [&](uint64_t s) {
        const uint64_t t = tiles * s, waves = (t + sms - 1) / sms;
        return (double)waves * ((double)kb / (double)s + 12.0) + 0.07 * (double)t;
    };
    int best = 1;
    double best_cost = cost(1);
    for (int s = 2; s <= 64; s++) {
        if (kb % s != 0 || K / s < 512) continue;
        const double c = cost((uint64_t)s);
        if (c < best_cost * 0.97) {
            best_cost = c;
            best = s;
        }
    }
    return best;
}

template <class T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int slices, size_t n, T* __restrict__ out) {
    const size_t nvec = n / 4, stride = (size_t)gridDim.x * 256;
    for (size_t v = (size_t)blockIdx.x * 256 + threadIdx.x; v < nvec; v += stride) {
        float4 acc = *reinterpret_cast<const float4*>(partial + 4 * v);
        for (int s = 1; s < slices; s++) {
            const float4 q = *reinterpret_cast<const float4*>(partial + (size_t)s * n + 4 * v);
            acc.x += q.x;
            acc.y += q.y;
            acc.z += q.z;
            acc.w += q.w;
        }
        if constexpr (std::is_same<T, float>::value) {
            *reinterpret_cast<float4*>(out + 4 * v) = acc;
        } else {
            Vec<T, 4> o;
            o.v[0] = from_f32<T>(acc.x);
            o.v[1] = from_f32<T>(acc.y);
            o.v[2] = from_f32<T>(acc.z);
            o.v[3] = from_f32<T>(acc.w);
            *reinterpret_cast<Vec<T, 4>*>(out + 4 * v) = o;
        }
    }
}

void splitk_reduce(int dtype, const float* partial, int slices, size_t n, void* out, const char* where) {
    // n is a multiple of 4 here: the tensor-core path requires N to be a multiple of 16 bytes' worth of elements
    size_t blocks = (n / 4 + 255) / 256;
    const size_t cap = (size_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (dtype == 0) splitk_reduce_kernel<bf16><<<(unsigned)blocks, 256, 0, ctx().stream>>>(partial, slices, n, static_cast<bf16*>(out));
    else if (dtype == 1) splitk_reduce_kernel<f16><<<(unsigned)blocks, 256, 0, ctx().stream>>>(partial, slices, n, static_cast<f16*>(out));
    else splitk_reduce_kernel<float><<<(unsigned)blocks, 256, 0, ctx().stream>>>(partial, slices, n, static_cast<float*>(out));
    check_launch(where);
}

namespace {
struct DeviceState {
    int* err = nullptr;     // device error word
    int seq = 0;            // launches made so far (the tag of a launch is seq & 0x7FFFFF, never 0)
    bool unchecked = false; // a launch was made since the host last read the word
};
thread_local DeviceState t_state[64];

DeviceState* current_state() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return &t_state[dev];
}
}  // namespace

int* next_launch_error_word(int* tag) {
    DeviceState* s = current_state();
    if (!s) return nullptr;
    if (!s->err) {
        if (cudaMalloc(&s->err, sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            s->err = nullptr;
            return nullptr;
        }
        cudaMemset(s->err, 0, sizeof(int));
    }
    s->seq = (s->seq + 1) & 0x7FFFFF;
    if (s->seq == 0) s->seq = 1;
    s->unchecked = true;
    *tag = s->seq;
    return s->err;
}

WaitReport next_wait_report() {
    WaitReport w;
    w.tag = 0;
    w.err = next_launch_error_word(&w.tag);
    return w;
}

}  // namespace tc

// Reads the error word of the calling thread's device.  The copy runs on the legacy stream, i.e. after the work the
// thread has queued there; call it after a synchronisation point.  A non-zero word sets the sticky status
// kErrDeviceWait (its detail = the code of the wait that gave up) and is cleared.
static int collect_tc_status(bool only_if_unchecked) {
    tc::DeviceState* s = tc::current_state();
    if (!s || !s->err) return 0;
    if (only_if_unchecked && !s->unchecked) return 0;
    int v = 0;
    if (cudaMemcpy(&v, s->err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    s->unchecked = false;
    if (v != 0) {
        set_error(kErrDeviceWait, v & 0xFF, (v & 0xFF) >= 21 ? "staged elementwise / conv kernel" : "tc_gemm_kernel");
        cudaMemset(s->err, 0, sizeof(int));
    }
    return v & 0xFF;
}

// Called by the ABI's own synchronisation points (cuda_memcpy_d2h, cuda_stream_synchronize): costs one 4-byte
// read-back, and only when a tensor-core launch was made since the last check.
int tc_status_after_sync() { return collect_tc_status(true); }

}  // namespace mx

// Checks the error word of the calling thread's device after a synchronisation point: 0 = fine, else the code of
// the bounded wait that ran out (also recorded as the sticky status kErrDeviceWait).
extern "C" int mx_tc_gemm_status(void) { return mx::collect_tc_status(false); }

// Test hook: writes `value` into the error word the way a kernel of an EARLIER launch would have left it
// (tag 0 is never handed to a launch), so the surfacing of a stale report can be tested without making a wait run out.
extern "C" int mx_debug_tc_gemm_poke_status(int value) {
    int tag = 0;
    int* err = mx::tc::next_launch_error_word(&tag);
    if (!err) return -1;
    const int word = value ? (value & 0xFF) | (0x7FFFFF << 8) : 0;
    return cudaMemcpy(err, &word, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
}

namespace mx {

// TMA wants 16-byte aligned bases and row pitches: the contiguous extent of every matrix (K for K-major
// operands, MN for MN-major ones, N for D) must be a multiple of 16 / elem_size elements.
static bool eligible(size_t es, uint64_t M, uint64_t N, uint64_t K, uint64_t batch, bool a_mn, bool b_mn, const void* a, const void* b, const void* d) {
    const uint64_t q = 16 / es;
    if (M == 0 || N == 0 || K == 0) return false;
    if (N % q != 0) return false;
    if ((a_mn ? M : K) % q != 0 || (b_mn ? N : K) % q != 0) return false;
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)d) % 16 != 0) return false;
    if (M > 0x7FFFFFFFull || N > 0x7FFFFFFFull || K > 0x7FFFFFFFull) return false;
    if (batch > 1 && (M * N) % q != 0) return false;  // every batch's output starts on a 16-byte boundary
    if (batch * M * N * K < (1ull << 24)) return false;  // small problems are not worth a persistent launch
    if (batch * ((M + 127) / 128) * ((N + 127) / 128) > 0x3FFFFFFFull) return false;
    return true;
}

// Forward product C[m, n] = sum_k A[m, k] * B[k, n]: can it run on a tensor-core kernel, and with which operand
// majors?  Unbatched, every operand either dense row-major or the transposed view of a dense matrix.
static bool classify_forward(const MmDesc& d, size_t es, size_t num_els, const void* x, const void* y, const void* out, TcProduct& c) {
    if (d.out_nd < 2 || d.a_nd < 2 || d.b_nd < 2) return false;
    const uint64_t m = d.m, n = d.n, k = d.k_fwd;
    if (m == 0 || n == 0 || num_els % (m * n) != 0) return false;
    const uint64_t batch = num_els / (m * n);
    // batched: rank-3 operands only (for higher ranks the reference indexes the batch through strides[0] alone)
    if (batch > 1 && !(d.out_nd == 3 && d.a_nd == 3 && d.b_nd == 3)) return false;
    if (batch > 0x7FFFull) return false;
    c.A = static_cast<const char*>(x) + d.a_off * es;
    c.B = static_cast<const char*>(y) + d.b_off * es;
    bool a_kmajor, a_mnmajor, b_kmajor, b_mnmajor;
    if (d.a_cont && d.b_cont) {
        // the reference's contiguous branch: A is [batch, m, k], B is [batch, k, n], both dense
        a_kmajor = true;
        a_mnmajor = false;
        b_kmajor = false;
        b_mnmajor = true;
        c.a_bs = (int64_t)(m * k);
        c.b_bs = (int64_t)(k * n);
    } else {
        // strided branch: A[b * as0 + m * as1 + k * as2], B[b * bs0 + k * bs1 + n * bs2]
        a_kmajor = d.a_strides[2] == 1 && d.a_strides[1] == (int64_t)k;
        a_mnmajor = d.a_strides[1] == 1 && d.a_strides[2] == (int64_t)m;  // transposed view of a dense [k, m] matrix
        b_kmajor = d.b_strides[1] == 1 && d.b_strides[2] == (int64_t)k;   // transposed view of a dense [n, k] matrix
        b_mnmajor = d.b_strides[2] == 1 && d.b_strides[1] == (int64_t)n;  // dense [k, n]
        c.a_bs = batch > 1 ? d.a_strides[0] : 0;                          // 0: one matrix broadcast over the batch
        c.b_bs = batch > 1 ? d.b_strides[0] : 0;
    }
    if (!(a_kmajor || a_mnmajor) || !(b_kmajor || b_mnmajor)) return false;
    if (batch > 1) {
        // a batch stride is a TMA stride: a multiple of 16 bytes, and whole matrices apart (no overlap tricks)
        const int64_t q = (int64_t)(16 / es);
        if (c.a_bs < 0 || c.b_bs < 0 || c.a_bs % q != 0 || c.b_bs % q != 0) return false;
        if ((c.a_bs != 0 && c.a_bs < (int64_t)(m * k)) || (c.b_bs != 0 && c.b_bs < (int64_t)(k * n))) return false;
    }
    c.a_mn = !a_kmajor;
    c.b_mn = !b_kmajor;
    c.m = m;
    c.n = n;
    c.k = k;
    c.batch = batch;
    return eligible(es, m, n, k, batch, c.a_mn, c.b_mn, c.A, c.B, out);
}

// which = 0: forward (x = A base, y = B base).  1: grad_a[m, k] = sum_n g[m, n] * B[k, n] (x = g, y = B + offset),
// reduction over n, both operands K-major.  2: grad_b[k, n] = sum_m A[m, k] * g[m, n] (x = g, y = A + offset),
// reduction over m, both operands MN-major.  The backward products read g, A and B as dense row-major matrices
// (strides ignored, crates/maidenx_cpu/src/ops/matmul.rs:196-261).
bool tc_classify(const MmDesc& d, int which, size_t es, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, const void* out,
                 TcProduct& c) {
    if (which == 0) return classify_forward(d, es, num_els, x, y, out, c);
    if (d.out_nd != 2) return false;
    const uint64_t m = d.m, n = d.n, k = d.k_bwd;
    if (d.g_size != m * n || nea != m * k || neb != k * n) return false;
    c.batch = 1;
    c.a_bs = c.b_bs = 0;
    if (which == 1) {
        c.A = static_cast<const char*>(x);
        c.B = static_cast<const char*>(y);
        c.a_mn = c.b_mn = false;
        c.m = m;
        c.n = k;
        c.k = n;
    } else {
        c.A = static_cast<const char*>(y);
        c.B = static_cast<const char*>(x);
        c.a_mn = c.b_mn = true;
        c.m = k;
        c.n = n;
        c.k = m;
    }
    return eligible(es, c.m, c.n, c.k, 1, c.a_mn, c.b_mn, c.A, c.B, out);
}

// x [rows, in] . w[out, in]^T with the bias add (and GELU) in the epilogue; false = shape not taken (the caller runs the ops one by one)
bool tc_linear_bias_act(bool is_bf16, uint64_t rows, uint64_t in_features, uint64_t out_features, const void* x, const void* w, const void* bias,
                        void* u, void* act, const char* where) {
    TcProduct c;
    c.A = static_cast<const char*>(x);
    c.B = static_cast<const char*>(w);
    c.a_mn = c.b_mn = false;
    c.m = rows;
    c.n = out_features;
    c.k = in_features;
    c.batch = 1;
    c.a_bs = c.b_bs = 0;
    if (!bias || !u || !eligible(2, c.m, c.n, c.k, 1, false, false, x, w, u) || (act && (uintptr_t)act % 16 != 0)) return false;
    return launch_gemm(is_bf16, c, u, where, act ? 2 : 1, bias, act);
}

// out[b] = w[rows, k] (shared by every batch) . cols[b][k, n] + bias[rows] broadcast along n, the bias add in the
// product's epilogue with the roundings of the two separate ops; false = shape not taken, nothing launched.
bool tc_batched_row_bias(bool is_bf16, uint64_t batch, uint64_t rows, uint64_t k, uint64_t n, const void* w, const void* cols, const void* bias, void* out,
                         const char* where) {
    TcProduct c;
    c.A = static_cast<const char*>(w);
    c.B = static_cast<const char*>(cols);
    c.a_mn = false;
    c.b_mn = true;  // [k, n] row-major per batch
    c.m = rows;
    c.n = n;
    c.k = k;
    c.batch = batch;
    c.a_bs = 0;
    c.b_bs = (int64_t)(k * n);
    if (!bias || !out || batch == 0 || batch > 0x7FFFull || !eligible(2, c.m, c.n, c.k, batch, false, true, w, cols, out)) return false;
    return launch_gemm(is_bf16, c, out, where, 3, bias, nullptr);
}

bool tc_gemm_bf16_f16(bool is_bf16, const MmDesc& d, int which, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, void* out,
                      const char* where) {
    TcProduct c;
    if (!tc_classify(d, which, 2, num_els, nea, neb, x, y, out, c)) return false;
    return launch_gemm(is_bf16, c, out, where);
}

}  // namespace mx

// Host-only view for tests without a GPU: would cuda_matmul_<bf16|f16> with this HOST metadata and these base
// addresses run on the tensor-core kernel?  Returns 0 (SIMT kernel) or 1, and the operand majors (0 = K-major,
// 1 = MN-major) and extents it would be launched with.
static int debug_forward_path(size_t es, size_t num_els, const size_t* host_metadata, const void* a, const void* b, const void* out, int* a_mn_major,
                              int* b_mn_major, size_t* m, size_t* n, size_t* k) {
    mx::MmDesc d;
    if (!host_metadata || !mx::mm_parse(host_metadata, d)) return 0;
    mx::TcProduct c;
    if (!mx::tc_classify(d, 0, es, num_els, 0, 0, a, b, out, c)) return 0;
    if (a_mn_major) *a_mn_major = c.a_mn ? 1 : 0;
    if (b_mn_major) *b_mn_major = c.b_mn ? 1 : 0;
    if (m) *m = c.m;
    if (n) *n = c.n;
    if (k) *k = c.k;
    return (int)c.batch;
}
// 2: bf16 / f16 products run on the two-CTA kernel (pairs of SMs share the B tile); 1: on the one-CTA kernel.
extern "C" void mx_set_gemm_cta_group(int ctas) { mx::g_two_cta.store(ctas == 2, std::memory_order_relaxed); }
extern "C" int mx_debug_gemm_max_resident_pairs(void) { return mx::tc2::max_resident_pairs(); }
extern "C" void mx_debug_set_gemm_group_m(int rows) { mx::g_group_m.store(rows > 0 ? rows : 16, std::memory_order_relaxed); }
// 1 (default): products with a reduction of at most 256 run with the B panel resident in shared memory; 0: general schedule
extern "C" void mx_debug_set_gemm_keep_b(int on) { mx::g_keep_b.store(on ? 1 : 0, std::memory_order_relaxed); }
extern "C" int mx_debug_gemm_keep_b_ctas(int tiles_m, int tiles_n, int num_kb, int batch, int ctas) { return mx::keep_b_ctas(tiles_m, tiles_n, num_kb, batch, ctas); }
extern "C" int mx_debug_splitk_slices(size_t tiles, size_t k, int block_k, int sms) { return mx::tc::splitk_slices(tiles, k, block_k, sms); }
extern "C" int mx_debug_matmul_forward_path(size_t num_els, const size_t* host_metadata, const void* a, const void* b, const void* out, int* a_mn_major,
                                            int* b_mn_major, size_t* m, size_t* n, size_t* k) {
    return debug_forward_path(2, num_els, host_metadata, a, b, out, a_mn_major, b_mn_major, m, n, k);
}
extern "C" int mx_debug_matmul_forward_path_f32(size_t num_els, const size_t* host_metadata, const void* a, const void* b, const void* out,
                                                int* a_mn_major, int* b_mn_major, size_t* m, size_t* n, size_t* k) {
    return debug_forward_path(4, num_els, host_metadata, a, b, out, a_mn_major, b_mn_major, m, n, k);
}
