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
// Buffers are dense (the reference casts whole buffers); each thread converts one 16-byte vector of the
// source: HBM-bound, sizeof(from) + sizeof(to) bytes per element.
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

template <class From, class To>
__global__ void __launch_bounds__(kCastThreads) cast_kernel(const From* __restrict__ in, To* __restrict__ out, u64 n, int vector_ok) {
    constexpr int VEC = 16 / (int)sizeof(From);
    const u64 stride = (u64)gridDim.x * kCastThreads;
    const u64 nvec = vector_ok ? n / VEC : 0;
    for (u64 v = (u64)blockIdx.x * kCastThreads + threadIdx.x; v < nvec; v += stride) {
        const Vec<From, VEC> x = *reinterpret_cast<const Vec<From, VEC>*>(in + v * VEC);
        Vec<To, VEC> y;
#pragma unroll
        for (int j = 0; j < VEC; j++) y.v[j] = cast_one<From, To>(x.v[j]);
        // the destination vector is VEC * sizeof(To) bytes: stored in 16-byte pieces (or one smaller piece)
        constexpr int kBytes = VEC * (int)sizeof(To);
        if constexpr (kBytes >= 16) {
            const uint4* src = reinterpret_cast<const uint4*>(&y);
            uint4* dst = reinterpret_cast<uint4*>(out + v * VEC);
#pragma unroll
            for (int k = 0; k < kBytes / 16; k++) dst[k] = src[k];
        } else if constexpr (kBytes == 8) {
            *reinterpret_cast<uint2*>(out + v * VEC) = *reinterpret_cast<const uint2*>(&y);
        } else if constexpr (kBytes == 4) {
            *reinterpret_cast<uint32_t*>(out + v * VEC) = *reinterpret_cast<const uint32_t*>(&y);
        } else {
            *reinterpret_cast<uint16_t*>(out + v * VEC) = *reinterpret_cast<const uint16_t*>(&y);
        }
    }
    for (u64 i = nvec * VEC + (u64)blockIdx.x * kCastThreads + threadIdx.x; i < n; i += stride) out[i] = cast_one<From, To>(in[i]);
}

template <class From, class To>
void cast_entry(size_t n, const From* in, To* out, const char* where) {
    if (n == 0) return;
    constexpr int VEC = 16 / (int)sizeof(From);
    const bool vector_ok = ((uintptr_t)in) % 16 == 0 && ((uintptr_t)out) % (VEC * sizeof(To) >= 16 ? 16 : VEC * sizeof(To)) == 0;
    u64 blocks = (n / VEC + kCastThreads - 1) / kCastThreads;
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
