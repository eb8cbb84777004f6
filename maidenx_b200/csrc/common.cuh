// Shared host/device infrastructure of the sm_100a op library: element types, vector
// access helpers, 32-bit fast division, the per-thread launch context (device, stream,
// sticky error) and the metadata resolver that turns the C-ABI's metadata pointer
// (device memory in the reference's calling convention) into a host-side array.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <type_traits>

namespace mx {

typedef __nv_bfloat16 bf16;
typedef __half f16;
typedef float f32;
typedef double f64;
typedef uint8_t u8;
typedef uint16_t u16;
typedef uint32_t u32;
typedef uint64_t u64;
typedef int8_t i8;
typedef int16_t i16;
typedef int32_t i32;
typedef int64_t i64;

template <class T>
struct is_half : std::false_type {};
template <>
struct is_half<bf16> : std::true_type {};
template <>
struct is_half<f16> : std::true_type {};
template <class T>
constexpr bool is_half_v = is_half<T>::value;
template <class T>
constexpr bool is_bool_v = std::is_same<T, bool>::value;
template <class T>
constexpr bool is_fp_v = std::is_floating_point<T>::value;
template <class T>
constexpr bool is_int_v = std::is_integral<T>::value && !is_bool_v<T>;

__host__ __device__ inline float to_f32(bf16 v) { return __bfloat162float(v); }
__host__ __device__ inline float to_f32(f16 v) { return __half2float(v); }
template <class T>
__host__ __device__ inline T from_f32(float v);
template <>
__host__ __device__ inline bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }
template <>
__host__ __device__ inline f16 from_f32<f16>(float v) { return __float2half_rn(v); }

// ---------------------------------------------------------------------------------
// Vector access: N elements of T moved as one naturally-aligned access.
// ---------------------------------------------------------------------------------
template <class T, int N>
struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

// ---------------------------------------------------------------------------------
// Division of a 32-bit unsigned value by a runtime-constant divisor.
// q = (mulhi(n, m) + n) >> s, the sum taken in 64 bits so every n < 2^32 is exact.
// ---------------------------------------------------------------------------------
struct FastDiv {
    uint32_t d, m, s;
    FastDiv() : d(1), m(0), s(0) {}
    explicit FastDiv(uint32_t div) { init(div); }
    void init(uint32_t div) {
        d = div ? div : 1;
        s = 0;
        while ((1ull << s) < d) s++;
        m = (uint32_t)(((1ull << 32) * ((1ull << s) - d)) / d + 1);
    }
    __host__ __device__ inline uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
        return (uint32_t)(((uint64_t)__umulhi(n, m) + n) >> s);
#else
        return (uint32_t)(((((uint64_t)n * m) >> 32) + n) >> s);
#endif
    }
    __host__ __device__ inline void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
};

// ---------------------------------------------------------------------------------
// Launch context
// ---------------------------------------------------------------------------------
constexpr int kMaxDims = 8;  // after merging; larger ranks are rejected with an error status

enum Status : int {
    kOk = 0,
    kErrCuda = 1,         // a CUDA runtime call or launch failed (code in last_cuda_error)
    kErrBadMetadata = 2,  // metadata could not be read / rank too large
    kErrUnsupported = 3,  // shape or size outside what the kernels handle
    kErrNoDevice = 4,
    kErrDeviceWait = 5,   // a bounded device-side wait ran out
};

struct ThreadCtx {
    cudaStream_t stream = 0;  // legacy default stream unless mx_set_stream was called
    int status = kOk;         // sticky: first error since the last mx_clear_error
    int cuda_error = 0;
    char where[96] = {0};
    int gemm_sm_limit = 0;    // > 0: the tensor-core GEMM launches at most this many CTAs (SMs left free for a concurrent exchange kernel)
};
ThreadCtx& ctx();
void set_error(int status, int cuda_error, const char* where);
// Check cudaGetLastError after a launch; records a sticky error.
void check_launch(const char* where);

// Resolve the C-ABI metadata pointer to host memory.  `meta` may be (a) NULL,
// (b) device memory uploaded through cuda_memcpy_h2d (found in the side table without
// touching the GPU), (c) any other device memory (copied back with a synchronous
// cudaMemcpy) or (d) plain host memory (used as is).  `count` is the number of size_t
// words the op needs; the result is valid until the next call on this thread.
const size_t* resolve_metadata(const size_t* meta, size_t count);

// Scratch memory for multi-pass kernels: one growable buffer per host thread and device,
// used in stream order on the thread's current stream.
void* scratch(size_t bytes);

int sm_count();
// Blocks of `kernel` that stay resident on one SM at this block size and dynamic shared memory (at least 1).
int resident_blocks(const void* kernel, int threads, size_t dynamic_smem = 0);

inline uint32_t ceil_div_u32(uint64_t a, uint64_t b) { return (uint32_t)((a + b - 1) / b); }

}  // namespace mx
