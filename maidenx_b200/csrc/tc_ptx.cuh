// Inline-PTX building blocks shared by the tensor-core kernels (tcgen05.mma with TMEM accumulators,
// TMA loads and stores, mbarriers with bounded waits) and the host helpers they share: the
// cuTensorMapEncodeTiled entry point and the per-thread, per-device error word.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace mx {
namespace tc {

constexpr long long TC_WAIT_BUDGET_CYCLES = 4000000000ll;  // about two seconds

// ---------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Error word protocol.  One 32-bit word per host thread and device, shared by every launch of the
// tensor-core kernels: 0 = fine, else (launch tag << 8) | code of the wait that gave up.  A launch only
// reacts to a word that carries ITS OWN tag, so a word left behind by an earlier launch (not yet
// collected by the host) does not make later launches abandon their tiles.
__device__ __forceinline__ bool tc_err_mine(const int* err, int tag) {
    const int e = *reinterpret_cast<const volatile int*>(err);
    return e != 0 && (e >> 8) == tag;
}
__device__ __forceinline__ void tc_err_report(int* err, int tag, int code) {
    const int mine = (tag << 8) | code;
    const int old = atomicCAS(err, 0, mine);
    if (old != 0 && (old >> 8) != tag) atomicExch(err, mine);  // a stale report of an older launch gives way
}
// Where a kernel outside the GEMM family records that one of its bounded waits ran out: the same per-device error
// word, tagged with the launch.  err == nullptr (no word could be had): the kernel gives up silently as before.
struct WaitReport {
    int* err;
    int tag;
};
__device__ __forceinline__ void wait_gave_up(const WaitReport& w, int code) {
    if (w.err) tc_err_report(w.err, w.tag, code);
}

// Bounded wait: returns false (and records `code` in *err) when the budget runs out or when
// another thread of this launch has already reported an error.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int tag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (tc_err_mine(err, tag)) return false;
        if (clock64() - t0 > TC_WAIT_BUDGET_CYCLES) {
            tc_err_report(err, tag, code);
            return false;
        }
    }
}

// The same bounded wait for roles in which many threads wait at once (whole warps of splitter or epilogue threads):
// between polls the thread sleeps, so that a hundred spinning threads do not take shared-memory bandwidth and issue
// slots from the TMA writes and the tensor core's operand reads.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, int* err, int tag, int code, unsigned sleep_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; i++) {
            __nanosleep(sleep_ns);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (tc_err_mine(err, tag)) return false;
        if (clock64() - t0 > TC_WAIT_BUDGET_CYCLES) {
            tc_err_report(err, tag, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
// 3-d forms: the third coordinate is the batch index (extent 1 for unbatched products and broadcast operands)
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, tied to the registers a load fills: the values count as produced by this statement, so no use of them
// can be scheduled ahead of it while the load is still in flight.  reg_fence ties a second register block to the same point.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) : : "memory");
}
__device__ __forceinline__ void reg_fence(uint32_t (&r)[32]) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) : : "memory");
}

// Shared-memory matrix descriptors, 128-byte swizzle.  Fields: start address >> 4 in bits
// [0,14), leading byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor
// version 1 (sm_100) at bit 46, layout type 2 (128-byte swizzle) in [61,64).
//  * K-major tile (rows of 64 K-elements = 128 bytes): groups of 8 rows are 1024 bytes apart
//    (stride byte offset); the leading byte offset is not used.  Advancing 16 elements along K
//    stays inside the swizzled row: +32 bytes on the start address.
//  * MN-major tile, stored as chunks of [64 K-rows x 64 MN-elements] (one TMA box each, 8 KB):
//    groups of 8 K-rows are 1024 bytes apart (stride byte offset) and the next 64 MN-elements
//    start 8192 bytes later (leading byte offset).  Advancing 16 elements along K = two groups
//    of 8 K-rows: +2048 bytes on the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operands of 32-bit elements (tf32) use the 128-byte swizzle with a 32-byte atom (layout type 1; TMA's
// SWIZZLE_128B_ATOM_32B): 32-byte chunks of a 128-byte row are XOR-ed with the row index modulo 4, so the pattern
// repeats every four K-rows (512 bytes): the stride byte offset is the distance between groups of FOUR K-rows and the
// leading byte offset the distance between 128-byte-wide MN chunks.
__device__ __forceinline__ uint64_t smem_desc_sw128_atom32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

// ---------------------------------------------------------------------------------
// host side (defined in matmul_tc.cu)
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn();

// [rows, cols] row-major matrix of `elem_bytes`-wide elements; box = box_rows x (128 / elem_bytes) columns, 128-byte swizzle.
bool make_map_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// `batch` row-major [rows, cols] matrices `batch_stride` elements apart (0 = one matrix read by every batch:
// the map then has extent 1 along the third dimension and the kernel passes coordinate 0); box = box_rows x
// (128 / elem_bytes) columns x 1, 128-byte swizzle.
// `pitch` = elements between consecutive rows (0: dense, = cols).
bool make_map_3d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t rows, uint64_t cols, uint64_t batch,
                 uint64_t batch_stride, uint32_t box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, uint64_t pitch = 0);

// Split-K plan for a product with few output tiles and a long reduction: the K range is cut into `slices` equal parts
// that run as the batches of one launch (each operand's slice is a sub-matrix reachable through the tensor map: a column
// range of a K-major operand, a row range of an MN-major one), the f32 partial results [slices, M, N] go to scratch and
// splitk_reduce adds them up and rounds once.  Returns 1 when splitting does not pay.
int splitk_slices(uint64_t tiles, uint64_t K, int block_k, int sms);
// out[i] = round(sum_s partial[s * n + i]); dtype: 0 bf16, 1 f16, 2 f32.
void splitk_reduce(int dtype, const float* partial, int slices, size_t n, void* out, const char* where);

// The error word of the calling thread's current device (allocated on first use) and the tag of the launch about
// to be made.  Returns nullptr when there is no usable device.
int* next_launch_error_word(int* tag);
// The same word and a fresh tag as a WaitReport, for the staged elementwise / conv kernels (codes 21..23).
WaitReport next_wait_report();

}  // namespace tc
}  // namespace mx
