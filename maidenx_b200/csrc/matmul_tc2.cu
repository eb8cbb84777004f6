// Two-CTA form of the bf16 / f16 tensor-core GEMM: tcgen05.mma.cta_group::2.
//
// Two CTAs on neighbouring SMs (a cluster of two) compute one 256 x 256 output tile.  Each CTA stages its own 128
// rows of A and HALF of the B tile (128 of the 256 columns) per k-block - 32 KB instead of the 48 KB of the one-CTA
// kernel - and the pair's tensor cores read both halves of B (the other half comes over the cluster interconnect),
// so shared-memory fill and operand reads per flop drop by a third and the ring is six stages deep instead of four.
// Each CTA accumulates its own 128 x 256 half of the tile in its own TMEM and runs its own epilogue.
//
// Roles per CTA (192 threads): warp 0 lane 0 = TMA producer (both CTAs; the loads carry .cta_group::2 and signal the
// LEADER's "full" barrier, whose transaction count covers both CTAs' bytes), warp 1 lane 0 of the leader (cluster rank
// 0) = MMA issuer for the pair, warps 2-5 = epilogue (TMEM -> registers -> swizzled staging -> TMA store).
// Cross-CTA signalling uses plain forms only: the leader commits every stage and every finished accumulator twice,
// once to its own barrier and once to the peer's barrier (a shared::cluster address), and the peer's epilogue warps
// arrive remotely on the leader's "accumulator free" barrier.  No cluster-scope loads, no multicast of any kind.
// Every mbarrier wait is bounded (tc_ptx.cuh); the two cluster barriers (after set-up, before TMEM is freed) are reached
// by every thread on every path.
#include <cuda.h>

#include <mutex>

#include "matmul_tc2.cuh"
#include "tc_ptx.cuh"

namespace mx {
namespace tc2 {

using namespace tc;

namespace {

constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KB: this CTA's 128 rows
constexpr int B_STAGE_BYTES = BN_HALF * BK * 2;   // 16 KB: this CTA's 128 of the 256 columns
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_WARPS = 4;
constexpr int EPI_CHUNK_COLS = 64;
constexpr int EPI_STAGE_BYTES = 32 * EPI_CHUNK_COLS * 2;  // 4 KB per warp per buffer
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = 512;                    // two 256-column f32 accumulators per CTA
constexpr int GROUP_PAIRS = 8;                    // row-tile pairs per column sweep (16 row tiles, as the one-CTA kernel)
constexpr int MN_CHUNK_BYTES = 64 * BK * 2;       // one [64 K-rows x 64 MN] box

struct Smem {
    static constexpr int a = 0;
    static constexpr int b = a + STAGES * A_STAGE_BYTES;
    static constexpr int epi = b + STAGES * B_STAGE_BYTES;
    static constexpr int bars = epi + EPI_WARPS * 2 * EPI_STAGE_BYTES;
    static constexpr int total = bars + 256;
};
constexpr int SMEM_BYTES = Smem::total + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");

// kind::f16, f32 accumulation, M = 256 (the pair), N = 256
__host__ __device__ constexpr uint32_t make_idesc(bool is_bf16, bool a_mn_major, bool b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= (is_bf16 ? 1u : 0u) << 7;
    d |= (is_bf16 ? 1u : 0u) << 10;
    d |= (a_mn_major ? 1u : 0u) << 15;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(BN >> 3) << 17;
    d |= (uint32_t)((2 * BM) >> 4) << 24;
    return d;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared::cluster address of the location `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier at the shared::cluster address `bar` once every tcgen05.mma issued so far by this thread has
// completed in both CTAs.
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// TMA load of one box into THIS CTA's shared memory, completing bytes on the barrier at the shared::cluster address `bar`
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

// pair tile -> (row-tile pair, column tile, batch)
__device__ __forceinline__ void tile_coords(int tile, const Params& p, int& tmp, int& tn, int& tb) {
    tb = tile / p.tiles_per_batch;
    tile -= tb * p.tiles_per_batch;
    const int group_size = GROUP_PAIRS * p.tiles_n;
    const int group = tile / group_size;
    const int first = group * GROUP_PAIRS;
    const int rows = min(GROUP_PAIRS, p.tile_pairs_m - first);
    const int in_group = tile - group * group_size;
    tmp = first + in_group % rows;
    tn = in_group / rows;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
tc_gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_d,
                Params p, int* err, int tag) {
    extern __shared__ unsigned char tc2_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc2_smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + Smem::bars;
    // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM base word
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::bars + 8 * (2 * STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();     // 0 = leader
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);           // the leader's: its producer's arrive + both CTAs' bytes
            mbar_init(empty_bar(s), 1);          // one commit from the leader's MMA thread, in each CTA
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);          // one commit from the leader's MMA thread, in each CTA
            mbar_init(tempty_bar(a), 2 * EPI_WARPS);  // the leader's: the epilogue warps of both CTAs
        }
        fence_barrier_init();
    }
    if (warp == 1) {  // the same warp of both CTAs allocates the pair's tensor memory
        tmem_alloc2(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other CTA
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
                int tmp, tn, tb;
                tile_coords(tile, p, tmp, tn, tb);
                const int row0 = (2 * tmp + (int)rank) * BM;            // this CTA's rows of A and of the output
                const int col0 = tn * BN + (int)rank * BN_HALF;         // this CTA's half of the B tile
                const int za = p.a_batched ? tb : 0, zb = p.b_batched ? tb : 0;
                for (int kb = 0; kb < p.num_kb; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, err, tag, 1)) {
                        ok = false;
                        break;
                    }
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
                    const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
                    const uint32_t sa = smem_base + Smem::a + stage * A_STAGE_BYTES;
                    const uint32_t sb = smem_base + Smem::b + stage * B_STAGE_BYTES;
                    if (!p.a_mn) {
                        tma2_load_3d(sa, &map_a, kb * BK, row0, za, leader_full);
                    } else {
#pragma unroll
                        for (int h = 0; h < BM / 64; h++) tma2_load_3d(sa + h * MN_CHUNK_BYTES, &map_a, row0 + h * 64, kb * BK, za, leader_full);
                    }
                    if (!p.b_mn) {
                        tma2_load_3d(sb, &map_b, kb * BK, col0, zb, leader_full);
                    } else {
#pragma unroll
                        for (int h = 0; h < BN_HALF / 64; h++) tma2_load_3d(sb + h * MN_CHUNK_BYTES, &map_b, col0 + h * 64, kb * BK, zb, leader_full);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc(p.is_bf16 != 0, p.a_mn != 0, p.b_mn != 0);
            const uint32_t a_lbo = p.a_mn ? MN_CHUNK_BYTES : 16, b_lbo = p.b_mn ? MN_CHUNK_BYTES : 16;
            const uint64_t a_kstep = p.a_mn ? (2048 >> 4) : (32 >> 4), b_kstep = p.b_mn ? (2048 >> 4) : (32 >> 4);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, err, tag, 2)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
                for (int kb = 0; kb < p.num_kb; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, err, tag, 3)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = smem_desc_sw128(smem_base + Smem::a + stage * A_STAGE_BYTES, a_lbo, 1024);
                    const uint64_t db = smem_desc_sw128(smem_base + Smem::b + stage * B_STAGE_BYTES, b_lbo, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) umma2_f16(d_tmem, da + a_kstep * k, db + b_kstep * k, idesc, (kb | k) != 0);
                    // the stage may be refilled in BOTH CTAs once these MMAs have read it
                    umma2_commit(empty_bar(stage));
                    umma2_commit(map_to_cta(empty_bar(stage), 1));
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma2_commit(tfull_bar(acc));  // accumulator complete, in both CTAs' tensor memory
                umma2_commit(map_to_cta(tfull_bar(acc), 1));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int quarter = warp & 3;
        const int ew = warp - 2;
        unsigned char* stage_buf = smem + Smem::epi + ew * 2 * EPI_STAGE_BYTES;
        int acc = 0, buf = 0;
        uint32_t acc_phase = 0;
        for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
            int tmp, tn, tb;
            tile_coords(tile, p, tmp, tn, tb);
            const int row0 = (2 * tmp + (int)rank) * BM;
            const bool ready = mbar_wait(tfull_bar(acc), acc_phase, err, tag, 4);
            if (!__all_sync(0xFFFFFFFFu, ready)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / EPI_CHUNK_COLS; c++) {
                uint32_t v0[32], v1[32];
                tmem_ld_32x32b_x32(t_row + c * EPI_CHUNK_COLS, v0);
                tmem_ld_32x32b_x32(t_row + c * EPI_CHUNK_COLS + 32, v1);
                tmem_ld_wait();
                if (c == BN / EPI_CHUNK_COLS - 1) {
                    // every TMEM read of this accumulator is done: tell the leader's MMA thread
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
                }
                if (p.out_f32) {
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
                            tma_store_3d(&map_d, smem_u32(stage_buf + buf * EPI_STAGE_BYTES), tn * BN + c * EPI_CHUNK_COLS + h * 32, row0 + quarter * 32, tb);
                            tma_store_commit();
                        }
                        buf ^= 1;
                    }
                    continue;
                }
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
                    tma_store_3d(&map_d, smem_u32(stage_buf + buf * EPI_STAGE_BYTES), tn * BN + c * EPI_CHUNK_COLS, row0 + quarter * 32, tb);
                    tma_store_commit();
                }
                buf ^= 1;
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    // common exit: neither CTA may leave (its shared memory and barriers are the other's operands and signals) or free
    // the pair's tensor memory before both are done
    tc_fence_before();
    __syncthreads();
    if (tc_err_mine(err, tag)) {
        // a wait gave up: give bulk copies still in flight towards this CTA's shared memory time to land
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000ll) {
        }
        __syncthreads();
    }
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc2(tmem_base, TMEM_COLS);
    }
}

bool opt_in_shared_memory() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
        if (cudaFuncSetAttribute(tc_gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        done[dev] = true;
    }
    return true;
}

}  // namespace

// How many pairs of CTAs of this kernel can be resident at once on the current device (pairs must sit on SMs the
// hardware can join into a cluster, which can be fewer than half the SM count); -1 when the query fails.
int max_resident_pairs() {
    if (!opt_in_shared_memory()) return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, tc_gemm2_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return n;
}

bool launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, const Params& p, int ctas, int* err, int tag, cudaStream_t stream) {
    if (!opt_in_shared_memory()) return false;
    int grid = ctas & ~1;  // whole pairs
    if (grid > 2 * p.num_tiles) grid = 2 * p.num_tiles;
    if (grid < 2) return false;
    tc_gemm2_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ma, mb, md, p, err, tag);
    return true;
}

}  // namespace tc2
}  // namespace mx
