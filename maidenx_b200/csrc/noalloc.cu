// mx_sum_f32_noalloc: cuda_sum_f32 for callers that must not allocate.
//
// The regular reductions take their second-pass workspace from a cudaMalloc'ed scratch block
// that grows on demand.  Some callers cannot tolerate that: a latency-critical loop that has to
// stay free of driver allocation calls (cudaMalloc may block, cudaFree synchronises the device),
// a process that has handed all device memory to its own allocator, or code that runs where the
// allocating runtime calls are not permitted.  This entry point computes the same sum with the
// workspace in a fixed array that is part of the library image.
//
// Contract
//   * Arguments are those of cuda_sum_f32, except that `metadata` must be HOST memory
//     (nothing is copied or cached, so nothing is allocated on the host either).
//   * No cudaMalloc, cudaFree or other allocating call is made, on any path.
//   * The workspace is kNoAllocScratchBytes (1 MiB, plus 64 KiB of arrival counters for the
//     in-launch fold of split reductions) per GPU, reserved on every GPU that loads
//     the library for as long as the process lives.  A reduction whose partial results do not
//     fit is rejected: mx_last_error() == 3 (unsupported) and the output is left untouched.
//     (Rows/columns reductions need splits * outputs * 4 bytes; the scatter path, used for
//     several reduced dims or a non-contiguous input, needs outputs * 4 bytes.)
//   * The first call on each device does the set-up: it looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and queries the SM count and the kernels'
//     occupancy.  Make that first call before starting any stream capture.
//   * All calls share the array.  Every element a call reads was written by that same call
//     (partials are overwritten, the scatter workspace is re-initialised by its fill kernel),
//     so leftovers from earlier calls are harmless; but two calls that overlap on the GPU —
//     different streams, or different host threads on the same device — race on it.  Keep
//     calls to this entry point in one stream order per device.
#include <mutex>

#include "abi_common.cuh"
#include "reduction.cuh"

namespace mx {

namespace {

constexpr size_t kNoAllocScratchBytes = 1u << 20;
constexpr size_t kNoAllocCounters = 16384;  // u32 each, in front of the workspace; static storage starts zeroed
constexpr size_t kNoAllocCounterBytes = kNoAllocCounters * sizeof(u32);

// In host code this name is only a handle for the runtime's symbol table, not an address a
// kernel can use: the device address is obtained per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocCounterBytes + kNoAllocScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_addr[64] = {nullptr};

// Device address of the array on the current device; looked up once per device.
void* noalloc_scratch(const char* where) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error(kErrNoDevice, (int)e, where);
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            set_error(kErrCuda, (int)e, where);
            return nullptr;
        }
        g_scratch_addr[dev] = p;
    }
    return g_scratch_addr[dev];
}

}  // namespace

}  // namespace mx

using namespace mx;

extern "C" void mx_sum_f32_noalloc(size_t num_els, size_t num_dims, size_t num_red_dims, const size_t* metadata, const float* inp, float* out) {
    const char* where = "mx_sum_f32_noalloc";
    typedef RedTraits<f32, RED_SUM> TR;
    typedef TR::Acc Acc;
    constexpr int VEC = 4;
    if (!metadata) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, metadata) != cudaSuccess) {
        cudaGetLastError();
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    if (!(attr.type == cudaMemoryTypeUnregistered || attr.type == cudaMemoryTypeHost)) {  // must be readable here without a copy
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    RedPlan pl;
    red_plan_dims(pl, num_els, num_dims, num_red_dims, metadata);
    if (pl.kind == RP_EMPTY) return;
    if (pl.kind == RP_ERROR) {
        set_error(kErrBadMetadata, 0, where);
        return;
    }
    unsigned char* block = static_cast<unsigned char*>(noalloc_scratch(where));
    if (!block) return;
    u32* const all_counters = reinterpret_cast<u32*>(block);
    Acc* ws = reinterpret_cast<Acc*>(block + kNoAllocCounterBytes);
    const size_t ws_elems = kNoAllocScratchBytes / sizeof(Acc);
    cudaStream_t s = ctx().stream;
    const int sms = sm_count();
    inp += pl.off;
    const bool base_aligned = ((uintptr_t)inp) % 16 == 0;

    if (pl.kind == RP_ROWS) {
        const u64 O = pl.O, R = pl.R;
        const bool vec = base_aligned && R % VEC == 0;
        const u64 unit = (u64)kRedThreads * VEC * 4;
        // same split selection as cuda_sum_f32's block kernel; where cuda_sum_f32 would pick its per-thread or per-warp
        // kernels (very short rows, or many short rows) the two entry points add in a different order and agree
        // within the reduction tolerance, not bit for bit
        static int occ = 0;
        if (!occ) occ = resident_blocks((const void*)reduce_rows_block_kernel<f32, RED_SUM, VEC>, kRedThreads);
        u64 want = split_count(O, (u64)sms * occ);
        u64 max_splits = (R + unit - 1) / unit;
        u64 splits = want < max_splits ? want : max_splits;
        if (splits < 1) splits = 1;
        u64 seg = (R + splits - 1) / splits;
        seg = (seg + VEC - 1) / VEC * VEC;
        splits = (R + seg - 1) / seg;
        if (O > 65535) {  // beyond the grid's row limit: one warp per row, no workspace
            reduce_rows_warp_kernel<f32, RED_SUM, 1><<<(u32)((O + 7) / 8), kRedThreads, 0, s>>>(inp, out, O, R, pl.factor);
            check_launch(where);
            return;
        }
        if (O * splits > ws_elems) {  // partials would not fit: one block per row needs no workspace
            splits = 1;
            seg = (R + VEC - 1) / VEC * VEC;
        }
        u32* counters = splits > 1 && O <= kNoAllocCounters ? all_counters : nullptr;
        const int tree_fold = O <= 64 && splits >= 64;
        dim3 grid((u32)splits, (u32)O);
        if (vec) reduce_rows_block_kernel<f32, RED_SUM, VEC><<<grid, kRedThreads, 0, s>>>(inp, out, ws, R, seg, (u32)splits, pl.factor, counters, tree_fold);
        else reduce_rows_block_kernel<f32, RED_SUM, 1><<<grid, kRedThreads, 0, s>>>(inp, out, ws, R, seg, (u32)splits, pl.factor, counters, tree_fold);
        if (splits > 1 && !counters) {
            if (tree_fold) reduce_partials_block_kernel<f32, RED_SUM><<<(u32)O, kRedThreads, 0, s>>>(ws, out, (u32)splits, pl.factor);
            else reduce_partials_kernel<f32, RED_SUM><<<(u32)((O + kRedThreads - 1) / kRedThreads), kRedThreads, 0, s>>>(ws, out, O, (u32)splits, 0, pl.factor);
        }
        check_launch(where);
        return;
    }
    if (pl.kind == RP_COLS) {
        const u64 O = pl.O, R = pl.R, I = pl.I;
        const bool vec = base_aligned && I % VEC == 0;
        const int v = vec ? VEC : 1;
        u64 gx = (I + (u64)kColLanes * v - 1) / ((u64)kColLanes * v);
        u64 gz = O < 65535 ? O : 65535;
        static int occ = 0;
        if (!occ) occ = resident_blocks((const void*)reduce_cols_kernel<f32, RED_SUM, VEC>, kColLanes * kColRows);
        u64 want = split_count(gx * gz, (u64)sms * occ);
        u64 max_splits = (R + 63) / 64;
        u64 splits = want < max_splits ? want : max_splits;
        if (splits < 1) splits = 1;
        // shrink the split count until the partials fit the fixed workspace
        while (splits > 1 && splits * O * I > ws_elems) splits--;
        u64 seg = (R + splits - 1) / splits;
        splits = (R + seg - 1) / seg;
        u32* counters = splits > 1 && O * gx <= kNoAllocCounters ? all_counters : nullptr;
        dim3 grid((u32)gx, (u32)splits, (u32)gz);
        if (vec) reduce_cols_kernel<f32, RED_SUM, VEC><<<grid, kColLanes * kColRows, 0, s>>>(inp, out, ws, O, R, I, seg, (u32)splits, pl.factor, counters);
        else reduce_cols_kernel<f32, RED_SUM, 1><<<grid, kColLanes * kColRows, 0, s>>>(inp, out, ws, O, R, I, seg, (u32)splits, pl.factor, counters);
        if (splits > 1 && !counters) {
            u64 count = O * I;
            reduce_partials_kernel<f32, RED_SUM><<<(u32)((count + kRedThreads - 1) / kRedThreads), kRedThreads, 0, s>>>(ws, out, count, (u32)splits, 1, pl.factor);
        }
        check_launch(where);
        return;
    }
    // scatter path: one accumulator per output element
    if (pl.out_count > ws_elems) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    u32 fill_blocks = (u32)((pl.out_count + kRedThreads - 1) / kRedThreads);
    if (fill_blocks == 0) fill_blocks = 1;
    reduce_fill_kernel<f32, RED_SUM><<<fill_blocks, kRedThreads, 0, s>>>(ws, pl.out_count);  // the workspace must start from zero
    u64 sb = (pl.gen.n + kRedThreads - 1) / kRedThreads;
    if (sb > (u64)sms * 16) sb = (u64)sms * 16;
    if (sb) reduce_scatter_kernel<f32, RED_SUM><<<(u32)sb, kRedThreads, 0, s>>>(inp, ws, pl.gen);
    reduce_finalize_kernel<f32, RED_SUM><<<fill_blocks, kRedThreads, 0, s>>>(ws, out, pl.out_count, pl.factor);
    check_launch(where);
}
