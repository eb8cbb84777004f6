// Device functors for the elementwise families.  Semantics follow the CPU backend of
// the reference (the parity target), not its CUDA kernels, where the two differ:
// saturating integer add/sub/mul, defined division by zero, truncating integer sqrt,
// 16-bit float math carried out in f32 and rounded once.
//   binary lambdas:  crates/maidenx_cpu/src/ops/binary.rs:372-934
//   unary lambdas:   crates/maidenx_cpu/src/ops/unary.rs:124-741
#pragma once
#include <cfloat>
#include <climits>
#include <cmath>
#include <limits>

#include "common.cuh"

namespace mx {

template <class T>
__device__ __forceinline__ T zero_of() {
    if constexpr (is_half_v<T>) return from_f32<T>(0.0f);
    else return (T)0;
}

template <class T>
struct Lim {
    __device__ static constexpr T min() { return std::numeric_limits<T>::min(); }
    __device__ static constexpr T max() { return std::numeric_limits<T>::max(); }
};

// float -> integer with saturation and NaN -> 0 (the CPU backend's `as` casts)
template <class T, class F>
__device__ __forceinline__ T sat_cast(F v) {
    if (v != v) return (T)0;
    const F lo = (F)Lim<T>::min();
    // 2^(bits-1) (signed) or 2^bits (unsigned): exactly representable, unlike max()
    const F half_range = (F)(1ull << (sizeof(T) * 8 - 1));
    const F hi_excl = std::is_signed<T>::value ? half_range : half_range * (F)2;
    if (v <= lo) return Lim<T>::min();
    if (v >= hi_excl) return Lim<T>::max();
    return (T)v;
}

template <class T>
__device__ __forceinline__ T wrap_neg(T a) {
    typedef typename std::make_unsigned<T>::type U;
    return (T)(U)((U)0 - (U)a);
}
template <class T>
__device__ __forceinline__ T wrap_abs(T a) {
    return a < 0 ? wrap_neg(a) : a;
}
template <class T>
__device__ __forceinline__ T wrap_mul(T a, T b) {
    typedef typename std::make_unsigned<T>::type U;
    return (T)(U)((u64)(U)a * (u64)(U)b);
}
template <class T>
__device__ __forceinline__ T wrap_add(T a, T b) {
    typedef typename std::make_unsigned<T>::type U;
    return (T)(U)((U)a + (U)b);
}

template <class T>
__device__ __forceinline__ T sat_add(T a, T b) {
    if constexpr (sizeof(T) < 8) {
        i64 r = (i64)a + (i64)b;
        return r < (i64)Lim<T>::min() ? Lim<T>::min() : (r > (i64)Lim<T>::max() ? Lim<T>::max() : (T)r);
    } else if constexpr (std::is_signed<T>::value) {
        u64 r = (u64)a + (u64)b;
        // overflow iff operands share a sign that the result does not
        if ((((u64)a ^ r) & ((u64)b ^ r)) >> 63) return a < 0 ? Lim<T>::min() : Lim<T>::max();
        return (T)r;
    } else {
        u64 r = a + b;
        return r < a ? Lim<T>::max() : (T)r;
    }
}
template <class T>
__device__ __forceinline__ T sat_sub(T a, T b) {
    if constexpr (sizeof(T) < 8) {
        i64 r = (i64)a - (i64)b;
        return r < (i64)Lim<T>::min() ? Lim<T>::min() : (r > (i64)Lim<T>::max() ? Lim<T>::max() : (T)r);
    } else if constexpr (std::is_signed<T>::value) {
        u64 r = (u64)a - (u64)b;
        if ((((u64)a ^ (u64)b) & ((u64)a ^ r)) >> 63) return a < 0 ? Lim<T>::min() : Lim<T>::max();
        return (T)r;
    } else {
        return a < b ? (T)0 : (T)(a - b);
    }
}
template <class T>
__device__ __forceinline__ T sat_mul(T a, T b) {
    if constexpr (sizeof(T) < 4) {
        i64 r = (i64)a * (i64)b;
        return r < (i64)Lim<T>::min() ? Lim<T>::min() : (r > (i64)Lim<T>::max() ? Lim<T>::max() : (T)r);
    } else if constexpr (sizeof(T) == 4) {
        if constexpr (std::is_signed<T>::value) {
            i64 r = (i64)a * (i64)b;
            return r < (i64)INT_MIN ? INT_MIN : (r > (i64)INT_MAX ? INT_MAX : (T)r);
        } else {
            u64 r = (u64)a * (u64)b;
            return r > 0xFFFFFFFFull ? 0xFFFFFFFFu : (T)r;
        }
    } else if constexpr (std::is_signed<T>::value) {
        i64 hi = __mul64hi(a, b);
        i64 lo = (i64)((u64)a * (u64)b);
        if (hi != (lo >> 63)) return ((a < 0) != (b < 0)) ? Lim<T>::min() : Lim<T>::max();
        return lo;
    } else {
        u64 hi = __umul64hi(a, b);
        return hi ? Lim<T>::max() : (T)(a * b);
    }
}
template <class T>
__device__ __forceinline__ T sat_div(T a, T b) {  // b != 0
    if constexpr (std::is_signed<T>::value) {
        if (a == Lim<T>::min() && b == (T)-1) return Lim<T>::max();
    }
    return (T)(a / b);
}

// x^c for integers with the result the CPU backend produces by going through a
// floating-point pow and a saturating cast: exact while the power fits the float
// format, rounded to nearest double in [2^53, 2^64), saturated beyond.
template <class T>
__device__ __forceinline__ T int_pow(T x, T c) {
    typedef typename std::make_unsigned<T>::type U;
    bool neg_base = false, neg_exp = false;
    u64 base, e;
    if constexpr (std::is_signed<T>::value) {
        neg_base = x < 0;
        neg_exp = c < 0;
        base = neg_base ? (u64)0 - (u64)(i64)x : (u64)x;
        e = neg_exp ? (u64)0 - (u64)(i64)c : (u64)c;
    } else {
        base = (u64)x;
        e = (u64)c;
    }
    bool odd = e & 1;
    if (e == 0) return (T)1;  // pow(x, 0) == 1 for every x, NaN-free here
    if (neg_exp) {
        if (base == 0) return Lim<T>::max();              // pow(0, -n) = +inf
        if (base == 1) return (neg_base && odd) ? (T)-1 : (T)1;
        return (T)0;                                      // |result| < 1 truncates to 0
    }
    if (base == 0) return (T)0;
    if (base == 1) return (neg_base && odd) ? (T)-1 : (T)1;
    // base >= 2: at most 64 multiplications before overflowing 2^64
    u64 r = 1;
    bool overflow = false;
    if (e > 64) overflow = true;
    else
        for (u64 i = 0; i < e; i++) {
            if (__umul64hi(r, base)) {
                overflow = true;
                break;
            }
            r *= base;
        }
    bool negative = neg_base && odd;
    if (overflow) return negative ? Lim<T>::min() : Lim<T>::max();
    if constexpr (sizeof(T) == 8) {
        f64 d = __ull2double_rn(r);
        if (negative) d = -d;
        return sat_cast<T, f64>(d);
    } else {
        if (negative) return r > (u64)1 << (sizeof(T) * 8 - 1) ? Lim<T>::min() : (T)(U)((u64)0 - r);
        return r > (u64)Lim<T>::max() ? Lim<T>::max() : (T)r;
    }
}

// ------------------------------------------------------------------ float helpers
template <class T, class F32Fn, class F64Fn>
__device__ __forceinline__ T fp_apply(T x, F32Fn f32fn, F64Fn f64fn) {
    if constexpr (is_half_v<T>) return from_f32<T>(f32fn(to_f32(x)));
    else if constexpr (std::is_same<T, f32>::value) return f32fn(x);
    else return f64fn(x);
}
template <class T>
__device__ __forceinline__ bool fgt(T a, T b) {
    if constexpr (is_half_v<T>) return to_f32(a) > to_f32(b);
    else return a > b;
}
template <class T>
__device__ __forceinline__ bool flt(T a, T b) {
    if constexpr (is_half_v<T>) return to_f32(a) < to_f32(b);
    else return a < b;
}
template <class T>
__device__ __forceinline__ bool feq(T a, T b) {
    if constexpr (is_half_v<T>) return to_f32(a) == to_f32(b);
    else return a == b;
}
template <class T>
__device__ __forceinline__ bool truthy(T a) {
    return !feq(a, zero_of<T>());
}

// For bf16 / f16 every arithmetic functor below is "convert to f32, compute, round once".
// HalfCore<Op> exposes that f32 computation on its own so that the vector kernels can convert
// and round two elements per instruction (packed cvt) instead of going through the 16-bit
// element type one value at a time.  The result is identical by construction.
template <class Op>
struct HalfCore {
    static constexpr bool ok = false;
};
#define MX_HALF_CORE1(OP, EXPR)                                      \
    template <>                                                      \
    struct HalfCore<OP> {                                            \
        static constexpr bool ok = true;                             \
        __device__ __forceinline__ static f32 f(f32 v) { return EXPR; } \
    };
#define MX_HALF_CORE2(OP, EXPR)                                             \
    template <>                                                             \
    struct HalfCore<OP> {                                                   \
        static constexpr bool ok = true;                                    \
        __device__ __forceinline__ static f32 f(f32 a, f32 b) { return EXPR; } \
    };

// Division of 16-bit floats.  The CPU backend divides in f32 and rounds once to T; x / 0 is 0 for
// 0 / 0 and +inf otherwise.  half_div_exact is that definition, kept out of line.
template <class T>
__device__ __noinline__ T half_div_exact(T a, T b) {
    const f32 x = to_f32(a), y = to_f32(b);
    if (y == 0.0f) return from_f32<T>(x == 0.0f ? 0.0f : INFINITY);
    return from_f32<T>(x / y);
}

// Fast path: q = a * rcp(b), within 2 f32 ulp of the true quotient.  Rounding q to T gives the
// reference's bits whenever no rounding boundary of T lies between q and the IEEE f32 quotient:
//   * A quotient of two p-bit significands that is dyadic has at most p bits, so it never sits
//     exactly on a midpoint of T; otherwise its distance to the nearest midpoint is at least
//     2^-(2p+1) relative.  For bf16 (p = 8) that is 2^-17, far above the 2^-22 error of q: the
//     fast result is always right.  For f16 (p = 11) the bound is 2^-23, so an f16 quotient whose
//     dropped 13 bits are within 2 ulp of the midpoint pattern is flagged.
//   * Zero, subnormal, infinite or NaN q (b = 0, subnormal or huge b, over/underflow, results in
//     T's subnormal range where the rounding position moves) is flagged.
// Flagged elements are recomputed with half_div_exact; bit `idx` of `mask` marks them.
template <class T>
__device__ __forceinline__ f32 half_div_fast(f32 a, f32 b, uint32_t& mask, int idx) {
    f32 r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(b));
    const f32 q = a * r;
    const uint32_t qb = __float_as_uint(q);
    constexpr bool kBf = std::is_same<T, bf16>::value;
    constexpr uint32_t kLo = kBf ? 0x0D800000u /* 2^-100 */ : 0x38800000u /* 2^-14 */;
    constexpr uint32_t kHi = 0x71800000u;  // 2^100
    bool bad = (qb << 1) - (kLo << 1) >= ((kHi - kLo) << 1);
    if constexpr (!kBf) bad = bad || ((qb << 19) - (0x0FFEu << 19)) <= (4u << 19);
    if (bad) mask |= 1u << idx;
    return q;
}

// ------------------------------------------------------------------ binary
struct OpAdd {
    template <class T>
    __device__ static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a | b;
        else if constexpr (is_int_v<T>) return sat_add(a, b);
        else if constexpr (is_half_v<T>) return from_f32<T>(to_f32(a) + to_f32(b));
        else return a + b;
    }
};
struct OpSub {
    template <class T>
    __device__ static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & b;
        else if constexpr (is_int_v<T>) return sat_sub(a, b);
        else if constexpr (is_half_v<T>) return from_f32<T>(to_f32(a) - to_f32(b));
        else return a - b;
    }
};
struct OpMul {
    template <class T>
    __device__ static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a ^ b;
        else if constexpr (is_int_v<T>) return sat_mul(a, b);
        else if constexpr (is_half_v<T>) return from_f32<T>(to_f32(a) * to_f32(b));
        else return a * b;
    }
};
struct OpDiv {
    template <class T>
    __device__ static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & b;
        else if constexpr (is_int_v<T>) {
            if (b == 0) {
                if (a == 0) return (T)0;
                if constexpr (std::is_signed<T>::value) {
                    if (a < 0) return Lim<T>::min();
                }
                return Lim<T>::max();
            }
            return sat_div(a, b);
        } else if constexpr (is_half_v<T>) {
            return half_div_exact<T>(a, b);
        } else {
            if (b == (T)0) return a == (T)0 ? (T)0 : (T)INFINITY;
            return a / b;
        }
    }
};
struct OpMax {
    template <class T>
    __device__ static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a | b;
        else if constexpr (std::is_same<T, f32>::value) return fmaxf(a, b);
        else if constexpr (std::is_same<T, f64>::value) return fmax(a, b);
        else return fgt(a, b) ? a : b;
    }
};
struct OpMin {
    template <class T>
    __device__ static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & b;
        else if constexpr (std::is_same<T, f32>::value) return fminf(a, b);
        else if constexpr (std::is_same<T, f64>::value) return fmin(a, b);
        else return flt(a, b) ? a : b;
    }
};
struct OpEq {
    template <class T>
    __device__ static bool f(T a, T b) { return feq(a, b); }
};
struct OpNe {
    template <class T>
    __device__ static bool f(T a, T b) { return !feq(a, b); }
};
struct OpLt {
    template <class T>
    __device__ static bool f(T a, T b) {
        if constexpr (is_bool_v<T>) return !a & b;
        else return flt(a, b);
    }
};
struct OpLe {
    template <class T>
    __device__ static bool f(T a, T b) {
        if constexpr (is_bool_v<T>) return a <= b;
        else return flt(a, b) || feq(a, b);
    }
};
struct OpGt {
    template <class T>
    __device__ static bool f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & !b;
        else return fgt(a, b);
    }
};
struct OpGe {
    template <class T>
    __device__ static bool f(T a, T b) {
        if constexpr (is_bool_v<T>) return a >= b;
        else return fgt(a, b) || feq(a, b);
    }
};
struct OpLAnd {
    template <class T>
    __device__ static bool f(T a, T b) { return truthy(a) && truthy(b); }
};
struct OpLOr {
    template <class T>
    __device__ static bool f(T a, T b) { return truthy(a) || truthy(b); }
};
struct OpLXor {
    template <class T>
    __device__ static bool f(T a, T b) { return truthy(a) != truthy(b); }
};

// ------------------------------------------------------------------ unary
// EXPRH is what bf16 / f16 evaluate (in f32, rounded once).  Where it differs from EXPR32 it uses
// the hardware exp2 / reciprocal approximations: their error (a few f32 ulp) is three orders
// below the 16-bit rounding step, and the ops stay memory-bound instead of instruction-bound.
#define MX_FP_UNARY(NAME, EXPR32, EXPR64, EXPRH)                                                                     \
    struct NAME {                                                                                                    \
        template <class T>                                                                                           \
        __device__ static T f(T x) {                                                                                 \
            if constexpr (is_half_v<T>) {                                                                            \
                const f32 v = to_f32(x);                                                                             \
                return from_f32<T>(EXPRH);                                                                           \
            } else {                                                                                                 \
                return fp_apply(x, [](f32 v) -> f32 { return EXPR32; }, [](f64 v) -> f64 { return EXPR64; });         \
            }                                                                                                        \
        }                                                                                                            \
    };                                                                                                               \
    MX_HALF_CORE1(NAME, EXPRH)
MX_FP_UNARY(OpSigmoid, 1.0f / (1.0f + expf(-v)), 1.0 / (1.0 + exp(-v)), __fdividef(1.0f, 1.0f + __expf(-v)))
MX_FP_UNARY(OpTanh, tanhf(v), tanh(v), tanhf(v))
MX_FP_UNARY(OpSin, sinf(v), sin(v), sinf(v))
MX_FP_UNARY(OpCos, cosf(v), cos(v), cosf(v))
MX_FP_UNARY(OpTan, tanf(v), tan(v), tanf(v))
MX_FP_UNARY(OpLn, logf(v), log(v), logf(v))
MX_FP_UNARY(OpLog10, log10f(v), log10(v), log10f(v))
MX_FP_UNARY(OpLog2, log2f(v), log2(v), log2f(v))
MX_FP_UNARY(OpExp, expf(v), exp(v), __expf(v))
MX_FP_UNARY(OpExp10, powf(10.0f, v), pow(10.0, v), powf(10.0f, v))
MX_FP_UNARY(OpExp2, exp2f(v), exp2(v), exp2f(v))
MX_FP_UNARY(OpSoftplus, logf(1.0f + expf(v)), log(1.0 + exp(v)), logf(1.0f + expf(v)))
MX_FP_UNARY(OpRecip, 1.0f / v, 1.0 / v, 1.0f / v)
MX_FP_UNARY(OpSqrtF, sqrtf(v), sqrt(v), sqrtf(v))
MX_FP_UNARY(OpAbsF, fabsf(v), fabs(v), fabsf(v))
#undef MX_FP_UNARY

__device__ __forceinline__ f64 gelu_f64(f64 x) {
    const f64 s = 0.7978845608028654, c = 0.044715;
    f64 t = s * (x + c * x * x * x);
    return 0.5 * x * (1.0 + tanh(t));
}
// f32 and 16-bit outputs evaluate the same function as x * sigmoid(2t): 0.5 * (1 + tanh(t))
// == 1 / (1 + exp(-2t)).  With the hardware exp2 / reciprocal its error is below 1e-6 * |x| (no
// cancellation for negative x): a tenth of the f32 tolerance against the tanh form, three orders
// below the bf16 / f16 rounding step, and it costs a third of tanhf, which keeps the strided
// kernels memory-bound.  f64 keeps the tanh form.
__device__ __forceinline__ f32 gelu_f32_fast(f32 x) {
    // exp(-2t) = 2^(x * (k1 + k2 x^2)), k1 = -2 log2(e) sqrt(2/pi), k2 = 0.044715 k1
    const f32 k1 = -2.302208198f, k2 = -0.102943240f;
    f32 e;
    const f32 arg = x * fmaf(k2, x * x, k1);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(arg));
    return __fdividef(x, 1.0f + e);
}
struct OpGelu {
    template <class T>
    __device__ static T f(T x) {
        if constexpr (is_half_v<T>) return from_f32<T>(gelu_f32_fast(to_f32(x)));
        else return fp_apply(x, [](f32 v) { return gelu_f32_fast(v); }, [](f64 v) { return gelu_f64(v); });
    }
};
struct OpIdentity {  // the strided-to-dense copy behind mx_contiguous_<T>
    template <class T>
    __device__ static T f(T x) {
        return x;
    }
};
struct OpNeg {
    template <class T>
    __device__ static T f(T x) {
        if constexpr (is_int_v<T>) return wrap_neg(x);
        else if constexpr (is_half_v<T>) return from_f32<T>(-to_f32(x));
        else return -x;
    }
};
struct OpAbs {
    template <class T>
    __device__ static T f(T x) {
        if constexpr (is_int_v<T>) return wrap_abs(x);
        else return OpAbsF::f(x);
    }
};
struct OpSign {
    template <class T>
    __device__ static T f(T x) {
        if constexpr (is_half_v<T>) {
            f32 v = to_f32(x);
            return from_f32<T>(v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f));
        } else if constexpr (std::is_unsigned<T>::value) return x > 0 ? (T)1 : (T)0;
        else return x > 0 ? (T)1 : (x < 0 ? (T)-1 : (T)0);
    }
};
struct OpSquare {
    template <class T>
    __device__ static T f(T x) {
        if constexpr (is_int_v<T>) return wrap_mul(x, x);
        else if constexpr (is_half_v<T>) return from_f32<T>(to_f32(x) * to_f32(x));
        else return x * x;
    }
};
struct OpSqrt {
    template <class T>
    __device__ static T f(T x) {
        // |MIN| wraps back to MIN: the CPU backend then takes sqrt of a negative number, and the
        // NaN casts to 0.  Tested on x itself so the compiler cannot fold it into abs().
        if constexpr (is_int_v<T> && std::is_signed<T>::value) {
            if (x == Lim<T>::min()) return (T)0;
        }
        if constexpr (std::is_same<T, i64>::value) return sat_cast<T, f64>(sqrt(__ll2double_rn(wrap_abs(x))));
        else if constexpr (std::is_same<T, u64>::value) return sat_cast<T, f32>(sqrtf(__ull2float_rn(x)));
        else if constexpr (is_int_v<T> && std::is_signed<T>::value) return sat_cast<T, f32>(sqrtf((f32)wrap_abs(x)));
        else if constexpr (is_int_v<T>) return sat_cast<T, f32>(sqrtf((f32)x));
        else return OpSqrtF::f(x);
    }
};
struct OpRelu {
    template <class T>
    __device__ static T f(T x) { return fgt(x, zero_of<T>()) ? x : zero_of<T>(); }
};
struct OpLogicalNot {
    template <class T>
    __device__ static bool f(T x) {
        if constexpr (is_bool_v<T>) return !x;
        else return feq(x, zero_of<T>());
    }
};

// ------------------------------------------------------------------ unary with constant
struct OpPow {
    template <class T>
    __device__ static T f(T x, T c) {
        if constexpr (is_half_v<T>) return from_f32<T>(powf(to_f32(x), to_f32(c)));
        else if constexpr (std::is_same<T, f32>::value) return powf(x, c);
        else if constexpr (std::is_same<T, f64>::value) return pow(x, c);
        else return int_pow(x, c);
    }
};
struct OpLeakyRelu {
    template <class T>
    __device__ static T f(T x, T a) {
        if constexpr (is_half_v<T>) return to_f32(x) > 0.0f ? x : from_f32<T>(to_f32(a) * to_f32(x));
        else return x > (T)0 ? x : a * x;
    }
};
struct OpElu {
    template <class T>
    __device__ static T f(T x, T a) {
        if constexpr (is_half_v<T>) {
            f32 xf = to_f32(x);
            return xf > 0.0f ? x : from_f32<T>(to_f32(a) * (expf(xf) - 1.0f));
        } else if constexpr (std::is_same<T, f32>::value) return x > 0.0f ? x : a * (expf(x) - 1.0f);
        else return x > 0.0 ? x : a * (exp(x) - 1.0);
    }
};

MX_HALF_CORE2(OpAdd, a + b)
MX_HALF_CORE2(OpSub, a - b)
MX_HALF_CORE2(OpMul, a * b)
MX_HALF_CORE2(OpMax, a > b ? a : b)
MX_HALF_CORE2(OpMin, a < b ? a : b)
MX_HALF_CORE2(OpPow, powf(a, b))
MX_HALF_CORE2(OpLeakyRelu, a > 0.0f ? a : b * a)
MX_HALF_CORE2(OpElu, a > 0.0f ? a : b * (expf(a) - 1.0f))
MX_HALF_CORE1(OpGelu, gelu_f32_fast(v))
MX_HALF_CORE1(OpNeg, -v)
MX_HALF_CORE1(OpAbs, fabsf(v))
MX_HALF_CORE1(OpSquare, v * v)
MX_HALF_CORE1(OpSqrt, sqrtf(v))
MX_HALF_CORE1(OpRelu, v > 0.0f ? v : 0.0f)
MX_HALF_CORE1(OpSign, v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f))

// Sums and differences of two bf16 (or two f16) values: the exact result fits f32 whenever the
// operands' exponents are within 16 (13) bits, and otherwise the smaller operand is far below
// half an ulp of the larger, so "add in f32, round to T" and the hardware's correctly rounded
// packed add give the same bits.  One instruction per two elements.
template <class Op>
struct HalfNative {
    static constexpr bool ok = false;
};
template <>
struct HalfNative<OpAdd> {
    static constexpr bool ok = true;
    template <class T>
    __device__ __forceinline__ static uint32_t f(uint32_t a, uint32_t b) {
        if constexpr (std::is_same<T, bf16>::value) {
            __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
            return *reinterpret_cast<uint32_t*>(&r);
        } else {
            __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
            return *reinterpret_cast<uint32_t*>(&r);
        }
    }
};
template <>
struct HalfNative<OpSub> {
    static constexpr bool ok = true;
    template <class T>
    __device__ __forceinline__ static uint32_t f(uint32_t a, uint32_t b) {
        if constexpr (std::is_same<T, bf16>::value) {
            __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
            return *reinterpret_cast<uint32_t*>(&r);
        } else {
            __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
            return *reinterpret_cast<uint32_t*>(&r);
        }
    }
};

// Two 16-bit floats <-> two f32, one instruction each way where the hardware has it.
template <class T>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (std::is_same<T, bf16>::value) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <class T>
__device__ __forceinline__ uint32_t pack2_rn(f32 lo, f32 hi) {
    if constexpr (std::is_same<T, bf16>::value) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

// Adapters giving every family the call shape the kernels use.
template <class Op, class T, class O>
struct Binary {  // out = Op(a, b)
    static constexpr bool kCore = HalfCore<Op>::ok && is_half_v<T> && std::is_same<O, T>::value;
    static constexpr bool kNative = HalfNative<Op>::ok && is_half_v<T> && std::is_same<O, T>::value;
    // division of 16-bit floats: fast quotient per element, flagged elements redone exactly
    static constexpr bool kChecked = std::is_same<Op, OpDiv>::value && is_half_v<T> && std::is_same<O, T>::value;
    __device__ __forceinline__ O operator()(T a, T b) const { return (O)Op::template f<T>(a, b); }
    __device__ __forceinline__ f32 core(f32 a, f32 b) const { return HalfCore<Op>::f(a, b); }
    __device__ __forceinline__ f32 core_checked(f32 a, f32 b, uint32_t& mask, int idx) const {
        if constexpr (kChecked) return half_div_fast<T>(a, b, mask, idx);
        else return 0.0f;
    }
    __device__ __forceinline__ uint32_t native(uint32_t a, uint32_t b) const { return HalfNative<Op>::template f<T>(a, b); }
};
template <class Op, class T, class O>
struct Unary {  // out = Op(a)
    static constexpr bool kNative = false;
    static constexpr bool kChecked = false;
    static constexpr bool kCore = HalfCore<Op>::ok && is_half_v<T> && std::is_same<O, T>::value;
    __device__ __forceinline__ O operator()(T a) const { return (O)Op::template f<T>(a); }
    __device__ __forceinline__ f32 core(f32 a) const { return HalfCore<Op>::f(a); }
};
template <class Op, class T, class O>
struct UnaryConst {  // out = Op(a, c)
    static constexpr bool kNative = false;
    static constexpr bool kChecked = std::is_same<Op, OpDiv>::value && is_half_v<T> && std::is_same<O, T>::value;
    static constexpr bool kCore = HalfCore<Op>::ok && is_half_v<T> && std::is_same<O, T>::value;
    T c;
    __device__ __forceinline__ O operator()(T a) const { return (O)Op::template f<T>(a, c); }
    __device__ __forceinline__ f32 core(f32 a) const {
        if constexpr (is_half_v<T>) return HalfCore<Op>::f(a, to_f32(c));
        else return 0.0f;
    }
    __device__ __forceinline__ f32 core_checked(f32 a, uint32_t& mask, int idx) const {
        if constexpr (kChecked) return half_div_fast<T>(a, to_f32(c), mask, idx);
        else return 0.0f;
    }
};

}  // namespace mx
