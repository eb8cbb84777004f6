// Runtime half of the C ABI: the cudart wrappers the reference's Rust crate exports
// (crates/maidenx_cuda/src/lib.rs:38-163), the per-thread launch context, the metadata
// side table and the scratch allocator.
//
// Metadata side table.  The reference's dispatch layer uploads each op's dims/strides
// block with cuda_malloc + cuda_memcpy_h2d right before the call and frees it right
// after (crates/maidenx_core/src/be/ops/binary.rs:112-133,161-163), so the launcher
// would have to read device memory back just to size its grid.  Because those wrappers
// live in this library, cuda_memcpy_h2d remembers small uploads keyed by destination
// address; the op entry points find the block there without touching the GPU.  Blocks
// uploaded some other way are read back with a synchronous cudaMemcpy, and a metadata
// pointer that is ordinary host memory is used directly.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "maidenx_cuda.h"

namespace mx {

int tc_status_after_sync();  // matmul_tc.cu

namespace {
constexpr size_t kSideTableMaxBytes = 2048;

std::mutex g_meta_mutex;
std::unordered_map<const void*, std::vector<size_t>> g_meta_table;

struct ScratchSlot {
    void* ptr = nullptr;
    size_t bytes = 0;
};
thread_local ScratchSlot t_scratch[64];
thread_local std::vector<size_t> t_meta_copy;
thread_local ThreadCtx t_ctx;

int g_sm_count[64] = {0};
}  // namespace

ThreadCtx& ctx() { return t_ctx; }

void set_error(int status, int cuda_error, const char* where) {
    ThreadCtx& c = t_ctx;
    if (c.status != kOk) return;  // sticky: keep the first
    c.status = status;
    c.cuda_error = cuda_error;
    std::snprintf(c.where, sizeof(c.where), "%s", where ? where : "");
}

void check_launch(const char* where) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) set_error(kErrCuda, (int)e, where);
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

const size_t* resolve_metadata(const size_t* meta, size_t count) {
    if (!meta) return nullptr;
    {
        std::lock_guard<std::mutex> lk(g_meta_mutex);
        auto it = g_meta_table.find(meta);
        if (it != g_meta_table.end() && it->second.size() >= count) {
            t_meta_copy = it->second;
            return t_meta_copy.data();
        }
    }
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, meta);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error(kErrBadMetadata, (int)e, "resolve_metadata");
        return nullptr;
    }
    if (attr.type == cudaMemoryTypeUnregistered || attr.type == cudaMemoryTypeHost) return meta;
    t_meta_copy.resize(count);
    // Synchronous on purpose: ordered after prior work on the legacy stream, as the
    // reference's own cudaMemcpy-based uploads are.
    e = cudaMemcpy(t_meta_copy.data(), meta, count * sizeof(size_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        set_error(kErrBadMetadata, (int)e, "resolve_metadata");
        return nullptr;
    }
    return t_meta_copy.data();
}

int resident_blocks(const void* kernel, int threads, size_t dynamic_smem) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dynamic_smem) != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = 1;
    }
    return n;
}

// Arrival counters of the split reductions: kArrivalCounters zeroed words per host thread and
// device, allocated on first use.  The kernels leave them zeroed.
constexpr size_t kArrivalCounters = 16384;
thread_local uint32_t* t_counters[64] = {nullptr};

uint32_t* arrival_counters(uint64_t count) {
    if (count > kArrivalCounters) return nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!t_counters[dev]) {
        void* p = nullptr;
        if (cudaMalloc(&p, kArrivalCounters * sizeof(uint32_t)) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;  // the caller folds in a second launch instead
        }
        if (cudaMemset(p, 0, kArrivalCounters * sizeof(uint32_t)) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(p);
            return nullptr;
        }
        t_counters[dev] = static_cast<uint32_t*>(p);
    }
    return t_counters[dev];
}

void* scratch(size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_error(kErrNoDevice, 0, "scratch");
        return nullptr;
    }
    ScratchSlot& s = t_scratch[dev];
    if (s.bytes >= bytes && s.ptr) return s.ptr;
    size_t want = bytes < (size_t)(8u << 20) ? (size_t)(8u << 20) : bytes + bytes / 4;
    if (s.ptr) {
        // cudaFree synchronises the device, so earlier kernels that used the old block are done.
        cudaFree(s.ptr);
        s.ptr = nullptr;
        s.bytes = 0;
    }
    cudaError_t e = cudaMalloc(&s.ptr, want);
    if (e != cudaSuccess) {
        s.ptr = nullptr;
        set_error(kErrCuda, (int)e, "scratch");
        return nullptr;
    }
    s.bytes = want;
    return s.ptr;
}

static void side_table_forget(const void* p) {
    std::lock_guard<std::mutex> lk(g_meta_mutex);
    if (!g_meta_table.empty()) g_meta_table.erase(p);
}

}  // namespace mx

using namespace mx;

namespace mx {
namespace {
constexpr size_t kPoolSlotBytes = 2048;
constexpr size_t kPoolSlabSlots = 256;
std::atomic<bool> g_pool_enabled{true};

struct Slab {
    char* base;
    int device;
};
std::mutex g_pool_mutex;
std::vector<Slab> g_slabs;
std::vector<void*> g_free_slots[64];  // per device

void* pool_take() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_pool_mutex);
    std::vector<void*>& fl = g_free_slots[dev];
    if (fl.empty()) {
        void* slab = nullptr;
        if (cudaMalloc(&slab, kPoolSlotBytes * kPoolSlabSlots) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;  // the caller falls back to a plain allocation
        }
        g_slabs.push_back({static_cast<char*>(slab), dev});
        for (size_t i = kPoolSlabSlots; i-- > 0;) fl.push_back(static_cast<char*>(slab) + i * kPoolSlotBytes);
    }
    void* p = fl.back();
    fl.pop_back();
    return p;
}

bool pool_give_back(void* ptr) {
    if (!ptr) return false;
    std::lock_guard<std::mutex> lk(g_pool_mutex);
    for (const Slab& sl : g_slabs) {
        if (ptr >= sl.base && ptr < sl.base + kPoolSlotBytes * kPoolSlabSlots) {
            g_free_slots[sl.device].push_back(ptr);
            return true;
        }
    }
    return false;
}
}  // namespace
}  // namespace mx
using namespace mx;

extern "C" {

// Small blocks come from a pool.  The reference's dispatch layer allocates and frees a metadata block
// around EVERY op call (crates/maidenx_core/src/be/ops/binary.rs:112-133,161-163), and cudaFree
// synchronises the device each time; requests of up to kPoolSlotBytes are served from slabs of
// fixed-size slots that are handed back to a free list instead.  Reuse is safe in stream order: a
// slot is only rewritten by work queued after its previous user.  mx_set_small_pool(0) turns it off.
int cuda_malloc(void** ptr, size_t size) {
    if (ptr && size <= kPoolSlotBytes && g_pool_enabled.load(std::memory_order_relaxed)) {
        if (void* p = pool_take()) {
            *ptr = p;
            return (int)cudaSuccess;
        }
    }
    return (int)cudaMalloc(ptr, size);
}

int cuda_free(void* ptr) {
    side_table_forget(ptr);
    if (pool_give_back(ptr)) return (int)cudaSuccess;
    return (int)cudaFree(ptr);
}

void mx_set_small_pool(int enabled) { g_pool_enabled.store(enabled != 0, std::memory_order_relaxed); }

int cuda_memcpy_h2d(void* dst, const void* src, size_t size) {
    cudaError_t e = cudaMemcpy(dst, src, size, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && size > 0 && size <= kSideTableMaxBytes && size % sizeof(size_t) == 0) {
        std::vector<size_t> v(size / sizeof(size_t));
        std::memcpy(v.data(), src, size);
        std::lock_guard<std::mutex> lk(g_meta_mutex);
        g_meta_table[dst] = std::move(v);
    } else {
        side_table_forget(dst);
    }
    return (int)e;
}

// The reference's callers learn of device-side trouble only through the return codes of the copies and
// synchronisations that follow an op (the ops return void).  A tensor-core kernel whose bounded waits ran out is
// therefore reported here: sticky status kErrDeviceWait and a non-zero return (cudaErrorLaunchTimeout).
static int surface_device_waits(int e) {
    if (e == (int)cudaSuccess && mx::tc_status_after_sync() > 0) return (int)cudaErrorLaunchTimeout;
    return e;
}

int cuda_memcpy_d2h(void* dst, const void* src, size_t size) { return surface_device_waits((int)cudaMemcpy(dst, src, size, cudaMemcpyDeviceToHost)); }

int cuda_memcpy_d2d(void* dst, const void* src, size_t size) {
    side_table_forget(dst);
    return (int)cudaMemcpy(dst, src, size, cudaMemcpyDeviceToDevice);
}

int cuda_set_device(int device_id) { return (int)cudaSetDevice(device_id); }
int cuda_get_device(int* device_id) { return (int)cudaGetDevice(device_id); }
int cuda_stream_create(void** stream) { return (int)cudaStreamCreate(reinterpret_cast<cudaStream_t*>(stream)); }
int cuda_stream_destroy(void* stream) { return (int)cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream)); }
int cuda_stream_synchronize(void* stream) { return surface_device_waits((int)cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream))); }

int cuda_pointer_get_attributes(MxCudaPointerAttributes* attributes, const void* ptr) {
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, ptr);
    if (e == cudaSuccess && attributes) {
        attributes->type_ = (int)a.type;
        attributes->device = a.device;
        attributes->devicePointer = a.devicePointer;
        attributes->hostPointer = a.hostPointer;
    }
    return (int)e;
}

const char* cuda_error_string(int error_code) { return cudaGetErrorString((cudaError_t)error_code); }

// ---- additive exports ------------------------------------------------------------
void mx_set_gemm_sm_limit(int sms) { mx::ctx().gemm_sm_limit = sms > 0 ? sms : 0; }
void mx_set_stream(void* stream) { ctx().stream = reinterpret_cast<cudaStream_t>(stream); }
void* mx_get_stream(void) { return reinterpret_cast<void*>(ctx().stream); }
int mx_last_error(void) { return ctx().status; }
int mx_last_cuda_error(void) { return ctx().cuda_error; }
const char* mx_last_error_where(void) { return ctx().where; }
void mx_clear_error(void) {
    ThreadCtx& c = ctx();
    c.status = kOk;
    c.cuda_error = 0;
    c.where[0] = 0;
}
int mx_tc_gemm_status(void);
int mx_device_synchronize(void) {
    int e = (int)cudaDeviceSynchronize();
    if (e == 0) mx_tc_gemm_status();  // surfaces a tensor-core kernel whose bounded waits ran out
    return e;
}
int mx_metadata_table_size(void) {
    std::lock_guard<std::mutex> lk(g_meta_mutex);
    return (int)g_meta_table.size();
}

}  // extern "C"
