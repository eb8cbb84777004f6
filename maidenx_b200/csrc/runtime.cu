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
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "maidenx_cuda.h"

namespace mx {

int tc_status_after_sync();  // matmul_tc.cu

namespace {
constexpr size_t kSideTableMaxBytes = 2048;

// Side table, ordered by device address so that every recorded block overlapping a range can be dropped when that
// range is freed or overwritten through the wrappers.  It is a cache: a pointer that is not found is read back
// from the device, so dropping entries is always safe.  (A kernel that writes into a recorded block is not seen;
// the contract is the reference's own: a metadata block is uploaded with cuda_memcpy_h2d right before the call.)
constexpr size_t kSideTableMaxEntries = 1 << 16;
std::mutex g_meta_mutex;
std::map<uintptr_t, std::vector<size_t>> g_meta_table;

// drops every recorded block that overlaps [p, p + bytes); caller holds g_meta_mutex
void forget_range_locked(const void* p, size_t bytes) {
    if (g_meta_table.empty()) return;
    const uintptr_t lo = (uintptr_t)p, hi = lo + (bytes ? bytes : 1);
    auto it = g_meta_table.lower_bound(lo);
    if (it != g_meta_table.begin()) {
        auto prev = std::prev(it);
        if (prev->first + prev->second.size() * sizeof(size_t) > lo) it = prev;
    }
    while (it != g_meta_table.end() && it->first < hi) it = g_meta_table.erase(it);
}

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
        auto it = g_meta_table.find((uintptr_t)meta);
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

static void side_table_forget(const void* p, size_t bytes) {
    std::lock_guard<std::mutex> lk(g_meta_mutex);
    forget_range_locked(p, bytes);
}

}  // namespace mx

using namespace mx;

namespace mx {
namespace {
// ---------------------------------------------------------------------------------
// Caching allocator behind cuda_malloc / cuda_free.
//
// The reference's dispatch layer allocates and frees a metadata block around EVERY op call
// (crates/maidenx_core/src/be/ops/binary.rs:112-133,161-163) and its tensor layer allocates every op's output with
// cuda_malloc and drops it with cuda_free (crates/maidenx_core/src/buffer/cuda.rs:21-40,58-75); cudaFree synchronises
// the device each time, which dominates small workloads such as the README training example.  Requests of up to
// kPoolMaxBytes are therefore rounded up to a size class (2 KB slots carved from slabs for the metadata blocks,
// powers of two above that) and a freed block goes to its class's free list instead of back to the driver; at most
// kPoolCacheLimit bytes per device are kept, anything beyond is really freed.
//
// Reuse is ordered by the stream: a block is rewritten only by work queued after its previous user when everything
// runs on the legacy default stream (the reference's model) or on blocking streams.  A thread that launches on a
// stream of its own (mx_set_stream) gets an event recorded at cuda_free, and such a block is handed out again only
// once that event has completed - the cudaMemcpy wrappers run on the legacy stream, which does not wait for
// non-blocking streams.
// ---------------------------------------------------------------------------------
constexpr size_t kPoolSlotBytes = 2048;
constexpr size_t kPoolSlabSlots = 256;
constexpr size_t kPoolMaxBytes = (size_t)64 << 20;     // larger requests go straight to cudaMalloc / cudaFree
constexpr size_t kPoolCacheLimit = (size_t)2 << 30;    // cached (free) bytes kept per device
constexpr int kPoolClasses = 27;                       // class c holds blocks of 1 << c bytes (c = 12 .. 26); class 0 = slab slots
std::atomic<bool> g_pool_enabled{true};
std::atomic<bool> g_stage_enabled{true};

struct CachedBlock {
    void* ptr;
    cudaEvent_t done;  // null: freed in legacy-stream order, reusable at once
};
struct LiveBlock {
    int device;
    int cls;  // 0 = slab slot
};
struct Slab {
    char* base;
    int device;
};
std::mutex g_pool_mutex;
std::vector<Slab> g_slabs;
std::vector<CachedBlock> g_free[64][kPoolClasses];
std::unordered_map<void*, LiveBlock> g_live;  // blocks handed out by the pool (not the slab slots: those are found by range)
size_t g_cached_bytes[64] = {0};

int size_class(size_t size) {
    if (size <= kPoolSlotBytes) return 0;
    int c = 12;
    while (((size_t)1 << c) < size) c++;
    return c;
}

// Pops a reusable block of the class, skipping blocks whose last user on a non-blocking stream is still running.
void* take_cached(int dev, int cls) {
    std::vector<CachedBlock>& fl = g_free[dev][cls];
    for (size_t i = fl.size(); i-- > 0;) {
        if (fl[i].done) {
            if (cudaEventQuery(fl[i].done) != cudaSuccess) {
                cudaGetLastError();
                continue;
            }
            cudaEventDestroy(fl[i].done);
        }
        void* p = fl[i].ptr;
        fl[i] = fl.back();
        fl.pop_back();
        if (cls) g_cached_bytes[dev] -= (size_t)1 << cls;
        return p;
    }
    return nullptr;
}

// A cached block that carries no event was freed in legacy-stream order: work queued on the legacy stream (by any thread)
// may still read it.  A thread that launches on a non-blocking stream of its own is not ordered behind that work, so
// its stream is made to wait for everything queued on the legacy stream so far before it may touch the block.
thread_local cudaEvent_t t_legacy_mark[64] = {nullptr};
void order_after_legacy_stream(int dev, cudaStream_t user_stream) {
    if (user_stream == 0) return;
    if (!t_legacy_mark[dev] && cudaEventCreateWithFlags(&t_legacy_mark[dev], cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        t_legacy_mark[dev] = nullptr;
        cudaStreamSynchronize(0);
        return;
    }
    cudaEventRecord(t_legacy_mark[dev], 0);
    cudaStreamWaitEvent(user_stream, t_legacy_mark[dev], 0);
}

void* pool_take(size_t size) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    const int cls = size_class(size);
    void* reused = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_pool_mutex);
        reused = take_cached(dev, cls);
        if (reused && cls) g_live[reused] = {dev, cls};
    }
    if (reused) {
        order_after_legacy_stream(dev, ctx().stream);
        return reused;
    }
    std::lock_guard<std::mutex> lk(g_pool_mutex);
    if (cls == 0) {
        void* slab = nullptr;
        if (cudaMalloc(&slab, kPoolSlotBytes * kPoolSlabSlots) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;  // the caller falls back to a plain allocation
        }
        g_slabs.push_back({static_cast<char*>(slab), dev});
        std::vector<CachedBlock>& fl = g_free[dev][0];
        for (size_t i = kPoolSlabSlots; i-- > 1;) fl.push_back({static_cast<char*>(slab) + i * kPoolSlotBytes, nullptr});
        return slab;
    }
    void* p = nullptr;
    if (cudaMalloc(&p, (size_t)1 << cls) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    g_live[p] = {dev, cls};
    return p;
}

// 1: the block went back to a free list; 0: not a pool block; -1: a pool block that must really be freed (cache full).
// *bytes = the block's size when it is a pool block.
int pool_give_back(void* ptr, size_t* bytes) {
    *bytes = 0;
    if (!ptr) return 0;
    cudaStream_t user_stream = ctx().stream;
    std::lock_guard<std::mutex> lk(g_pool_mutex);
    int dev = -1, cls = -1;
    auto it = g_live.find(ptr);
    if (it != g_live.end()) {
        dev = it->second.device;
        cls = it->second.cls;
        g_live.erase(it);
        *bytes = (size_t)1 << cls;
        if (g_cached_bytes[dev] + ((size_t)1 << cls) > kPoolCacheLimit) return -1;
    } else {
        for (const Slab& sl : g_slabs)
            if (ptr >= sl.base && ptr < sl.base + kPoolSlotBytes * kPoolSlabSlots) {
                dev = sl.device;
                cls = 0;
                break;
            }
        if (cls < 0) return 0;
        *bytes = kPoolSlotBytes;
    }
    CachedBlock b{ptr, nullptr};
    if (user_stream != 0) {
        if (cudaEventCreateWithFlags(&b.done, cudaEventDisableTiming) == cudaSuccess) cudaEventRecord(b.done, user_stream);
        else {
            cudaGetLastError();
            b.done = nullptr;
            cudaStreamSynchronize(user_stream);  // no event to be had: make the block safe the slow way
        }
    }
    g_free[dev][cls].push_back(b);
    if (cls) g_cached_bytes[dev] += (size_t)1 << cls;
    return 1;
}
}  // namespace
}  // namespace mx
using namespace mx;

extern "C" {

int cuda_malloc(void** ptr, size_t size) {
    if (ptr && size <= kPoolMaxBytes && g_pool_enabled.load(std::memory_order_relaxed)) {
        if (void* p = pool_take(size)) {
            *ptr = p;
            return (int)cudaSuccess;
        }
    }
    return (int)cudaMalloc(ptr, size);
}

int cuda_free(void* ptr) {
    size_t bytes = 0;
    const int r = pool_give_back(ptr, &bytes);
    side_table_forget(ptr, bytes);  // every block recorded inside the freed allocation (its base alone when the size is unknown)
    if (r == 1) return (int)cudaSuccess;
    return (int)cudaFree(ptr);
}

// 0 turns the caching allocator off (every request goes to cudaMalloc / cudaFree, as in the reference); blocks
// already handed out are still recognised when they are freed.
void mx_set_small_pool(int enabled) {
    g_pool_enabled.store(enabled != 0, std::memory_order_relaxed);
    g_stage_enabled.store(enabled != 0, std::memory_order_relaxed);
}

// Small uploads (the per-call metadata blocks, scalars, tiny tensors) go through a per-thread ring of pinned
// staging slots and an asynchronous copy on the thread's current stream: a plain cudaMemcpy from pageable memory
// first waits for everything queued on the stream, which serialises host and device once per op call in the
// reference's dispatch pattern.  The source is copied into the slot before the call returns, so the caller may reuse
// it at once, and everything the thread queues afterwards (ops, the synchronous device-to-host copies) is ordered
// after the upload by the stream.  A slot is reused only after the event recorded behind its group has completed.
namespace {
constexpr size_t kStageSlotBytes = 2048;
constexpr int kStageSlots = 512, kStageGroup = 64;
struct StageRing {
    char* base = nullptr;
    cudaEvent_t done[kStageSlots / kStageGroup] = {nullptr};
    bool used[kStageSlots / kStageGroup] = {false};
    int next = 0;
    bool failed = false;
};
thread_local StageRing t_stage[64];

// Returns false when the staged path is unavailable (the caller then uses the synchronous copy).
bool staged_upload(void* dst, const void* src, size_t size, cudaError_t* result) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    StageRing& r = t_stage[dev];
    if (r.failed) return false;
    if (!r.base) {
        if (cudaHostAlloc(reinterpret_cast<void**>(&r.base), kStageSlotBytes * kStageSlots, cudaHostAllocDefault) != cudaSuccess) {
            cudaGetLastError();
            r.failed = true;
            return false;
        }
        for (auto& e : r.done)
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                r.failed = true;
                return false;
            }
    }
    const int slot = r.next, group = slot / kStageGroup;
    if (slot % kStageGroup == 0 && r.used[group]) cudaEventSynchronize(r.done[group]);  // the copies that last used this group have finished
    char* stage = r.base + (size_t)slot * kStageSlotBytes;
    std::memcpy(stage, src, size);
    cudaStream_t stream = ctx().stream;
    *result = cudaMemcpyAsync(dst, stage, size, cudaMemcpyHostToDevice, stream);
    r.next = (slot + 1) % kStageSlots;
    if (r.next % kStageGroup == 0) {
        cudaEventRecord(r.done[group], stream);
        r.used[group] = true;
    }
    return true;
}
}  // namespace

int cuda_memcpy_h2d(void* dst, const void* src, size_t size) {
    cudaError_t e;
    if (!(size > 0 && size <= kStageSlotBytes && g_stage_enabled.load(std::memory_order_relaxed) && staged_upload(dst, src, size, &e)))
        e = cudaMemcpy(dst, src, size, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && size > 0 && size <= kSideTableMaxBytes && size % sizeof(size_t) == 0) {
        std::vector<size_t> v(size / sizeof(size_t));
        std::memcpy(v.data(), src, size);
        std::lock_guard<std::mutex> lk(g_meta_mutex);
        forget_range_locked(dst, size);
        if (g_meta_table.size() >= kSideTableMaxEntries) g_meta_table.clear();
        g_meta_table[(uintptr_t)dst] = std::move(v);
    } else {
        side_table_forget(dst, size);
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

// The synchronous copies below run on the legacy stream, which does not wait for a non-blocking stream: when the
// thread launches on a stream of its own, its queued work (ops, staged uploads) is waited for first.
static void drain_thread_stream() {
    if (ctx().stream != 0) cudaStreamSynchronize(ctx().stream);
}

int cuda_memcpy_d2h(void* dst, const void* src, size_t size) {
    drain_thread_stream();
    return surface_device_waits((int)cudaMemcpy(dst, src, size, cudaMemcpyDeviceToHost));
}

int cuda_memcpy_d2d(void* dst, const void* src, size_t size) {
    drain_thread_stream();
    side_table_forget(dst, size);
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
