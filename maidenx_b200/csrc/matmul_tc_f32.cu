// Tensor-core path for f32 matmul on sm_100a: tcgen05.mma kind::tf32 with split operands, so the
// product keeps f32-level accuracy although the tensor core multiplies 11-bit significands.
//
// Every f32 operand element x is used as two tf32 values
//     big   = x with the low 13 significand bits dropped (what the tensor core reads from the raw f32 bits),
//     small = x - big   (exact in f32; its own low bits are again dropped by the tensor core),
// and each k-step issues three MMAs into the same TMEM accumulator:
//     a_small * b_big  +  a_big * b_small  +  a_big * b_big.
// The dropped term a_small * b_small and the truncation of `small` are each below 2^-21 of |a * b|, so a dot
// product agrees with f32 arithmetic to a few 1e-7 relative to sum |a_k * b_k| (the stated f32 matmul tolerance is
// 1e-4).
//
// Two-level accumulation.  The tensor core adds each instruction's products into the f32 accumulator with
// truncation, which pulls a long running sum towards zero by about half an ulp per instruction (measured:
// -6e-6 relative after 147 instructions); over K = 8192 that would eat the whole 1e-4 budget.  So the TMEM
// accumulator only ever holds the sum of CHUNK_KB k-blocks (128 values of K, 48 instructions): the epilogue warps
// drain it after every chunk and keep the running total in registers, added with round-to-nearest, while the tensor
// core fills the other accumulator.  The pull towards zero is then bounded by the chunk length (about -2e-6 of the
// result) whatever K is.
//
// One persistent CTA per SM, 320 threads in four roles:
//   warp 0      TMA producer: raw f32 A [128 x 32] and B [BN x 32] k-blocks (128-byte swizzle rows of 32 floats)
//               into a ring of STAGES stages;
//   warps 6-9   splitter: when a stage has landed, read the raw tiles and write the `small` tiles beside them
//               (element-wise, so the swizzled placement carries over unchanged), then hand the stage to
//   warp 1      the MMA issuer: 4 k-steps x 3 tcgen05.mma (M128, N = BN, K8) per k-block into one of two TMEM
//               accumulators, switching accumulator every CHUNK_KB k-blocks; commits the stage back to the
//               producer and each finished chunk to
//   warps 2-5   the epilogue: per chunk tcgen05.ld of the warp's 32 rows x BN columns, added into BN registers per
//               thread; after the tile's last chunk the totals go through a swizzled 4 KB staging tile to TMA stores.
// Operands may be K-major ([MN, K] row-major) or MN-major ([K, MN] row-major, loaded as [32 K-rows x 32 MN] boxes),
// which covers x . W^T, g . W and x^T . g without transposed copies.  No cluster launch, no multicast.
// Every mbarrier wait is bounded (see tc_ptx.cuh); on expiry all roles fall through to the common exit.
#include <cuda.h>

#include <mutex>

#include "matmul_tc.cuh"
#include "tc_ptx.cuh"

namespace mx {

using namespace tc;

namespace {

constexpr int BM = 128, BN = 128, BK = 32;     // CTA tile; BK * 4 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 8;                      // tf32: 32 bytes of K per instruction
constexpr int STAGES = 3;
constexpr int A_TILE = BM * BK * 4;            // 16 KB
constexpr int B_TILE = BN * BK * 4;
constexpr int RAW_BYTES = A_TILE + B_TILE;     // what TMA delivers per stage
constexpr int STAGE_BYTES = 2 * RAW_BYTES;     // [A raw | B raw | A small | B small]
constexpr int EPI_WARPS = 4, SPLIT_WARPS = 4;
constexpr int EPI_CHUNK_COLS = 32;             // 32 f32 = 128 bytes per staged row
constexpr int EPI_STAGE_BYTES = 32 * EPI_CHUNK_COLS * 4;  // 4 KB per warp per buffer
constexpr int THREADS = 32 * (2 + EPI_WARPS + SPLIT_WARPS);
constexpr int TMEM_COLS = 2 * BN;              // two f32 accumulators
constexpr int GROUP_M = 16;
constexpr int CHUNK_KB = 4;                    // k-blocks summed inside TMEM before the registers take over
constexpr int MN_CHUNK_BYTES = BK * 128;       // one [32 K-rows x 32 MN-elements] box

static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM allocations are powers of two");
static_assert(RAW_BYTES % (16 * 32 * SPLIT_WARPS) == 0, "the splitter moves 16 bytes per thread and step");

struct Smem {
    static constexpr int stages = 0;
    static constexpr int epi = stages + STAGES * STAGE_BYTES;
    static constexpr int bars = epi + EPI_WARPS * 2 * EPI_STAGE_BYTES;
    static constexpr int total = bars + 256;
};
constexpr int SMEM_BYTES = Smem::total + 1024;  // slack for the 1024-byte alignment
static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");

__host__ __device__ constexpr uint32_t make_idesc_tf32(bool a_mn_major, bool b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;                               // D format: f32
    d |= 2u << 7;                               // A format: tf32
    d |= 2u << 10;                              // B format: tf32
    d |= (a_mn_major ? 1u : 0u) << 15;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(BN >> 3) << 17;
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}

struct Params {
    int tiles_m, tiles_n, num_tiles, num_kb;
    int tiles_per_batch;       // tiles_m * tiles_n; num_tiles = batch * tiles_per_batch
    int a_batched, b_batched;  // 0: the operand is one matrix shared by every batch (third TMA coordinate stays 0)
    int a_mn, b_mn;
};

__device__ __forceinline__ void tile_coords(int tile, const Params& p, int& tm, int& tn, int& tb) {
    tb = tile / p.tiles_per_batch;
    tile -= tb * p.tiles_per_batch;
    const int group_size = GROUP_M * p.tiles_n;
    const int group = tile / group_size;
    const int first_m = group * GROUP_M;
    const int rows = min(GROUP_M, p.tiles_m - first_m);
    const int in_group = tile - group * group_size;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

// small = x - (x with its low 13 bits cleared), itself rounded to the 11 significant bits the tensor core will read
// (rounding here instead of letting the hardware truncate keeps the error of the split unbiased); infinities and
// NaNs keep all their weight in `big`.
__device__ __forceinline__ uint32_t small_part(uint32_t bits) {
    const float x = __uint_as_float(bits);
    const float big = __uint_as_float(bits & 0xFFFFE000u);
    const uint32_t s = (__float_as_uint(x - big) + 0x1000u) & 0xFFFFE000u;
    return (bits & 0x7F800000u) == 0x7F800000u ? 0u : s;
}

__global__ void __launch_bounds__(THREADS, 1)
tc_gemm_f32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_d,
                   Params p, int* err, int tag) {
    extern __shared__ unsigned char tcf_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tcf_smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + Smem::bars;
    // barrier slots (8 bytes each): full[STAGES], split[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM base word
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto split_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (3 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (3 * STAGES + 2 + a); };
    volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::bars + 8 * (3 * STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(split_bar(s), SPLIT_WARPS);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), EPI_WARPS);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
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
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                int tm, tn, tb;
                tile_coords(tile, p, tm, tn, tb);
                const int za = p.a_batched ? tb : 0, zb = p.b_batched ? tb : 0;
                for (int kb = 0; kb < p.num_kb; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, err, tag, 1)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full_bar(stage), RAW_BYTES);
                    const uint32_t sa = smem_base + Smem::stages + stage * STAGE_BYTES;
                    const uint32_t sb = sa + A_TILE;
                    if (!p.a_mn) {
                        tma_load_3d(sa, &map_a, kb * BK, tm * BM, za, full_bar(stage));
                    } else {
#pragma unroll
                        for (int h = 0; h < BM / 32; h++) tma_load_3d(sa + h * MN_CHUNK_BYTES, &map_a, tm * BM + h * 32, kb * BK, za, full_bar(stage));
                    }
                    if (!p.b_mn) {
                        tma_load_3d(sb, &map_b, kb * BK, tn * BN, zb, full_bar(stage));
                    } else {
#pragma unroll
                        for (int h = 0; h < BN / 32; h++) tma_load_3d(sb + h * MN_CHUNK_BYTES, &map_b, tn * BN + h * 32, kb * BK, zb, full_bar(stage));
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(p.a_mn != 0, p.b_mn != 0);
            // K-major: 8 floats further along the 128-byte row; MN-major: the next group of eight K-rows
            const uint64_t a_kstep = p.a_mn ? (1024 >> 4) : (32 >> 4), b_kstep = p.b_mn ? (1024 >> 4) : (32 >> 4);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += CHUNK_KB) {
                    if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, err, tag, 2)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
                    const int kb1 = min(kb0 + CHUNK_KB, p.num_kb);
                    for (int kb = kb0; kb < kb1; kb++) {
                        // the raw tiles (TMA) and the small tiles (splitter) are both operands
                        if (!mbar_wait(full_bar(stage), phase, err, tag, 3) || !mbar_wait(split_bar(stage), phase, err, tag, 6)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t s0 = smem_base + Smem::stages + stage * STAGE_BYTES;
                        // K-major: rows of 32 floats, groups of eight rows 1024 bytes apart.  MN-major: 32-byte-atom swizzle,
                        // groups of four K-rows 512 bytes apart, 128-byte-wide MN chunks one box (4 KB) apart.
                        const uint64_t a_big = p.a_mn ? smem_desc_sw128_atom32(s0, MN_CHUNK_BYTES, 512) : smem_desc_sw128(s0, 16, 1024);
                        const uint64_t b_big = p.b_mn ? smem_desc_sw128_atom32(s0 + A_TILE, MN_CHUNK_BYTES, 512) : smem_desc_sw128(s0 + A_TILE, 16, 1024);
                        const uint64_t a_small =
                            p.a_mn ? smem_desc_sw128_atom32(s0 + RAW_BYTES, MN_CHUNK_BYTES, 512) : smem_desc_sw128(s0 + RAW_BYTES, 16, 1024);
                        const uint64_t b_small = p.b_mn ? smem_desc_sw128_atom32(s0 + RAW_BYTES + A_TILE, MN_CHUNK_BYTES, 512)
                                                        : smem_desc_sw128(s0 + RAW_BYTES + A_TILE, 16, 1024);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++) {
                            umma_tf32(d_tmem, a_small + a_kstep * k, b_big + b_kstep * k, idesc, (kb != kb0) || (k != 0));
                            umma_tf32(d_tmem, a_big + a_kstep * k, b_small + b_kstep * k, idesc, 1);
                            umma_tf32(d_tmem, a_big + a_kstep * k, b_big + b_kstep * k, idesc, 1);
                        }
                        umma_commit(empty_bar(stage));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                    if (!ok) break;
                    umma_commit(tfull_bar(acc));  // this chunk's partial sums are complete
                    if (++acc == 2) {
                        acc = 0;
                        acc_phase ^= 1;
                    }
                }
            }
        }
    } else if (warp < 2 + EPI_WARPS) {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;  // TMEM lanes [32 * quarter, 32 * quarter + 32)
        const int ew = warp - 2;
        unsigned char* stage_buf = smem + Smem::epi + ew * 2 * EPI_STAGE_BYTES;
        int acc = 0, buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            int tm, tn, tb;
            tile_coords(tile, p, tm, tn, tb);
            float total[BN];  // this thread's row of the tile (registers: every index below is a compile-time constant)
#pragma unroll
            for (int j = 0; j < BN; j++) total[j] = 0.0f;
            for (int kb0 = 0; kb0 < p.num_kb; kb0 += CHUNK_KB) {
                // the TMEM loads below are warp-collective: leave the loops only as a whole warp
                const bool ready = mbar_wait_relaxed(tfull_bar(acc), acc_phase, err, tag, 4, 200);
                if (!__all_sync(0xFFFFFFFFu, ready)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
#pragma unroll
                for (int c = 0; c < BN / 32; c++) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(t_row + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) total[c * 32 + j] += __uint_as_float(v[j]);
                }
                // every TMEM read of this accumulator is done: hand it back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok) break;
#pragma unroll
            for (int c = 0; c < BN / EPI_CHUNK_COLS; c++) {
                // the staging buffer must have been read by its previous TMA store
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                unsigned char* dst = stage_buf + buf * EPI_STAGE_BYTES + lane * 128;  // row `lane` of the 32 x 32 tile
#pragma unroll
                for (int j = 0; j < 8; j++)  // eight 16-byte chunks per row, XOR-swizzled by the row index
                    *reinterpret_cast<float4*>(dst + ((j ^ (lane & 7)) << 4)) =
                        make_float4(total[c * 32 + 4 * j], total[c * 32 + 4 * j + 1], total[c * 32 + 4 * j + 2], total[c * 32 + 4 * j + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&map_d, smem_u32(stage_buf + buf * EPI_STAGE_BYTES), tn * BN + c * EPI_CHUNK_COLS, tm * BM + quarter * 32, tb);
                    tma_store_commit();
                }
                buf ^= 1;
            }
        }
        if (lane == 0) tma_store_wait_all();
    } else {
        // ------------------------------------------------------------ splitter (warps 6..9)
        const int t = threadIdx.x - 32 * (2 + EPI_WARPS);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < p.num_kb; kb++) {
                const bool landed = mbar_wait_relaxed(full_bar(stage), phase, err, tag, 5, 40);
                if (!__all_sync(0xFFFFFFFFu, landed)) {
                    ok = false;
                    break;
                }
                const uint4* raw = reinterpret_cast<const uint4*>(smem + Smem::stages + stage * STAGE_BYTES);
                uint4* small = reinterpret_cast<uint4*>(smem + Smem::stages + stage * STAGE_BYTES + RAW_BYTES);
                constexpr int STEPS = RAW_BYTES / 16 / (32 * SPLIT_WARPS);
#pragma unroll 8
                for (int i = 0; i < STEPS; i++) {
                    const uint4 q = raw[t + i * 32 * SPLIT_WARPS];
                    small[t + i * 32 * SPLIT_WARPS] = make_uint4(small_part(q.x), small_part(q.y), small_part(q.z), small_part(q.w));
                }
                fence_proxy_async_smem();  // the tensor core reads these through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(split_bar(stage));
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    }

    // common exit: TMEM is released by the warp that allocated it, after everyone is done with it
    tc_fence_before();
    __syncthreads();
    if (tc_err_mine(err, tag)) {
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

bool opt_in_shared_memory() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
        if (cudaFuncSetAttribute(tc_gemm_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        done[dev] = true;
    }
    return true;
}

// mn_major: the operand is loaded as [32 K-rows x 32 MN-elements] boxes in the 32-byte-atom form of the 128-byte swizzle
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t batch, uint64_t batch_stride, uint32_t box_rows,
              bool mn_major = false, uint64_t pitch = 0) {
    return make_map_3d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, rows, cols, batch, batch_stride, box_rows,
                       mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, pitch);
}

// D[M,N] = sum_k Aop[m,k] * Bop[n,k]; K-major operand = dense row-major [MN, K], MN-major = dense row-major [K, MN].
bool launch(const TcProduct& c, void* D, const char* where) {
    const void *A = c.A, *B = c.B;
    const bool a_mn = c.a_mn, b_mn = c.b_mn;
    const uint64_t M = c.m, N = c.n;
    uint64_t K = c.k, batch = c.batch;
    if (!opt_in_shared_memory()) return false;
    Params p;
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + BN - 1) / BN);
    p.tiles_per_batch = p.tiles_m * p.tiles_n;
    int grid = sm_count();
    if (ctx().gemm_sm_limit > 0 && ctx().gemm_sm_limit < grid) grid = ctx().gemm_sm_limit;
    // few output tiles, long reduction: cut K into slices that run as the batches of this launch (see tc_ptx.cuh)
    const int slices = batch == 1 ? splitk_slices((uint64_t)p.tiles_per_batch, K, BK, grid) : 1;
    float* partial = nullptr;
    uint64_t a_bs = (uint64_t)c.a_bs, b_bs = (uint64_t)c.b_bs, a_pitch = 0, b_pitch = 0;
    if (slices > 1) {
        partial = static_cast<float*>(scratch((size_t)slices * M * N * sizeof(float)));
        if (!partial) return false;
        const uint64_t Ks = K / slices;
        a_pitch = a_mn ? M : K;
        b_pitch = b_mn ? N : K;
        a_bs = a_mn ? Ks * M : Ks;
        b_bs = b_mn ? Ks * N : Ks;
        K = Ks;
        batch = (uint64_t)slices;
    }
    int tag = 0;
    int* err = next_launch_error_word(&tag);
    if (!err) return false;
    CUtensorMap ma, mb, md;
    const bool oka = a_mn ? make_map(&ma, A, K, M, batch, a_bs, BK, true, a_pitch) : make_map(&ma, A, M, K, batch, a_bs, BM, false, a_pitch);
    const bool okb = b_mn ? make_map(&mb, B, K, N, batch, b_bs, BK, true, b_pitch) : make_map(&mb, B, N, K, batch, b_bs, BN, false, b_pitch);
    if (!oka || !okb || !make_map(&md, partial ? static_cast<void*>(partial) : D, M, N, batch, M * N, 32)) return false;
    p.num_tiles = (int)batch * p.tiles_per_batch;
    p.a_batched = (batch > 1 && a_bs != 0) ? 1 : 0;
    p.b_batched = (batch > 1 && b_bs != 0) ? 1 : 0;
    p.num_kb = (int)((K + BK - 1) / BK);
    p.a_mn = a_mn ? 1 : 0;
    p.b_mn = b_mn ? 1 : 0;
    if (grid > p.num_tiles) grid = p.num_tiles;
    tc_gemm_f32_kernel<<<grid, THREADS, SMEM_BYTES, ctx().stream>>>(ma, mb, md, p, err, tag);
    check_launch(where);
    if (partial) splitk_reduce(2, partial, slices, (size_t)(M * N), D, where);
    return true;
}

}  // namespace

bool tc_gemm_f32(const MmDesc& d, int which, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, void* out, const char* where) {
    TcProduct c;
    if (!tc_classify(d, which, 4, num_els, nea, neb, x, y, out, c)) return false;
    return launch(c, out, where);
}

}  // namespace mx
