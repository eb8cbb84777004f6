// Device-side dtype casts (additive: mx_cast_<from>_<to>).  The reference converts between dtypes on
// the HOST even for CUDA buffers - copy out, map, copy back - in
// crates/maidenx_core/src/buffer/mod.rs:132-575 (copy_from_with_dtype_cast); these kernels apply the same
// element rules on the device:
//   16-bit float -> X        to_f32(x) `as` X (float -> int saturates, NaN -> 0); -> bool: to_f32(x) != 0
//   f32 / f64 -> 16-bit      from_f32(x as f32): an f64 is rounded to f32 first
//   f32 / f64 -> int, float  Rust `as`
//   anything -> bool         x != 0 (a NaN is true)
//   bool -> X                through u8 (0 / 1)
//   u8 / i8 -> 16-bit float  exact; wider integers -> 16-bit float keep only their low byte (`as u8` / `as i8`
//                            comes first in the reference)
//   int -> int               truncate or sign-/zero-extend
// Buffers are dense (the reference casts whole buffers): HBM-bound, sizeof(from) + sizeof(to) bytes per element.
#include "abi_common.cuh"
#include "ops.cuh"

namespace mx {

template <class From, class To>
__device__ __forceinline__ To cast_one(From x) {
    if constexpr (std::is_same<From, To>::value) {
        return x;
    } else if constexpr (std::is_same<To, bool>::value) {
        if constexpr (is_half_v<From>) return to_f32(x) != 0.0f;
        else return x != (From)0;
    } else if constexpr (is_half_v<From>) {
        const f32 v = to_f32(x);
        if constexpr (is_half_v<To>) return from_f32<To>(v);
        else if constexpr (std::is_floating_point<To>::value) return (To)v;
        else return sat_cast<To, f32>(v);
    } else if constexpr (is_half_v<To>) {
        if constexpr (std::is_floating_point<From>::value) return from_f32<To>((f32)x);
        else if constexpr (std::is_same<From, bool>::value) return from_f32<To>(x ? 1.0f : 0.0f);
        else if constexpr (std::is_signed<From>::value) return from_f32<To>((f32)(int8_t)x);
        else return from_f32<To>((f32)(uint8_t)x);
    } else if constexpr (std::is_floating_point<From>::value) {
        if constexpr (std::is_floating_point<To>::value) return (To)x;
        else return sat_cast<To, From>(x);
    } else if constexpr (std::is_same<From, bool>::value) {
        return (To)(uint8_t)(x ? 1 : 0);
    } else {
        return (To)x;
    }
}

constexpr int kCastThreads = 256;

// N bytes moved as one access (N a power of two, 1 .. 16)
template <int N>
struct CastWord;
template <>
struct CastWord<16> { typedef uint4 type; };
template <>
struct CastWord<8> { typedef uint2 type; };
template <>
struct CastWord<4> { typedef uint32_t type; };
template <>
struct CastWord<2> { typedef uint16_t type; };
template <>
struct CastWord<1> { typedef uint8_t type; };

// Each thread converts VEC = 16 / max(sizeof(From), sizeof(To)) elements per step, so that the WIDER side moves as
// full 16-byte vectors and the narrower side as one contiguous 8-, 4-, 2- or 1-byte piece per lane: every warp-level
// load and store is a dense run of bytes (a widening cast used to store two 16-byte halves 32 bytes apart per lane,
// which half-filled every sector it touched).  Four steps are in flight per thread.
template <class From, class To>
__global__ void __launch_bounds__(kCastThreads) cast_kernel(const From* __restrict__ in, To* __restrict__ out, u64 n, int vector_ok) {
    constexpr int WIDE = sizeof(From) > sizeof(To) ? (int)sizeof(From) : (int)sizeof(To);
    constexpr int VEC = 16 / WIDE;
    constexpr int UNROLL = 4;
    typedef typename CastWord<VEC * (int)sizeof(From)>::type InWord;
    typedef typename CastWord<VEC * (int)sizeof(To)>::type OutWord;
    const u64 stride = (u64)gridDim.x * kCastThreads;
    const u64 nvec = vector_ok ? n / VEC : 0;
    for (u64 v0 = (u64)blockIdx.x * kCastThreads + threadIdx.x; v0 < nvec; v0 += stride * UNROLL) {
        InWord x[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
            if (v0 + u * stride < nvec) x[u] = *reinterpret_cast<const InWord*>(in + (v0 + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            if (v0 + u * stride >= nvec) break;
            const From* xs = reinterpret_cast<const From*>(&x[u]);
            OutWord y;
            To* ys = reinterpret_cast<To*>(&y);
#pragma unroll
            for (int j = 0; j < VEC; j++) ys[j] = cast_one<From, To>(xs[j]);
            *reinterpret_cast<OutWord*>(out + (v0 + u * stride) * VEC) = y;
        }
    }
    for (u64 i = nvec * VEC + (u64)blockIdx.x * kCastThreads + threadIdx.x; i < n; i += stride) out[i] = cast_one<From, To>(in[i]);
}

template <class From, class To>
void cast_entry(size_t n, const From* in, To* out, const char* where) {
    if (n == 0) return;
    constexpr int WIDE = sizeof(From) > sizeof(To) ? (int)sizeof(From) : (int)sizeof(To);
    constexpr int VEC = 16 / WIDE;
    const bool vector_ok = ((uintptr_t)in) % (VEC * sizeof(From)) == 0 && ((uintptr_t)out) % (VEC * sizeof(To)) == 0;
    u64 blocks = (n / VEC + (u64)kCastThreads * 4 - 1) / ((u64)kCastThreads * 4);
    const u64 cap = (u64)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cast_kernel<From, To><<<(unsigned)blocks, kCastThreads, 0, ctx().stream>>>(in, out, (u64)n, vector_ok ? 1 : 0);
    check_launch(where);
}

}  // namespace mx

#define MX_DEF_CAST_(TO, FROM) \
    void mx_cast_##FROM##_##TO(size_t num_els, const mx_##FROM* in, mx_##TO* out) { mx::cast_entry<mx_##FROM, mx_##TO>(num_els, in, out, "mx_cast_" #FROM "_" #TO); }
#define MX_DEF_CAST(TO, FROM) MX_DEF_CAST_(TO, FROM)
#define MX_DEF_CAST_FROM(FROM, ...) MX_CAST_TARGETS(MX_DEF_CAST, FROM)

extern "C" {
MX_DTYPES_ALL(MX_DEF_CAST_FROM, _)
}
