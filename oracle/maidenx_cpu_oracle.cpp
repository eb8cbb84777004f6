// TEST INFRASTRUCTURE ONLY.
//
// CPU oracle: a C++ restatement of the reference's `maidenx_cpu` backend for the op
// layer (strided binary / unary elementwise, sum / sum_to_shape / mean / max / min,
// matmul / matmul_backward, conv2d im2col / col2im).  It exists to check the CUDA
// library and to provide the timed CPU baseline; the product library never links,
// loads or calls it.
//
// The reference backend is Rust and no Rust toolchain exists on the build or GPU
// machines, so the reference itself cannot be compiled; this file follows it function
// by function (citations are paths inside the reference project):
//   crates/maidenx_cpu/src/utils.rs:2-31            is_contiguous, get_strided_index
//   crates/maidenx_cpu/src/ops/binary.rs:13-248     binary / logical / in-place drivers
//   crates/maidenx_cpu/src/ops/binary.rs:372-934    per-dtype binary lambdas
//   crates/maidenx_cpu/src/ops/unary.rs:14-122      unary drivers
//   crates/maidenx_cpu/src/ops/unary.rs:124-741     per-dtype unary lambdas
//   crates/maidenx_cpu/src/ops/reduction.rs:6-272,383-625   sum, sum_to_shape, mean, max, min
//   crates/maidenx_cpu/src/ops/matmul.rs:5-296      matmul, matmul_backward
//   crates/maidenx_cpu/src/nn/conv.rs:13-158        im2col, col2im
// Exported symbols carry the reference backend's own names (`add_f32`, `sum_bf16`, …)
// and argument order, with the metadata pointer in host memory.
//
// Later sections add the rest of the backend with their own citations: fold, the three paddings with
// their backward passes, softmax, and the dtype casts of crates/maidenx_core/src/buffer/mod.rs.
//
// Pinning: checked against the known-answer vectors of the reference's own tests
// (crates/maidenx_tensor/tests/ops_{binary,unary,reduction,matmul,padding}.rs, the fold test in
// ops_reduction.rs, crates/maidenx_nn/src/losses/mse.rs), stored under tests/golden/.  The reference
// pins no values for im2col / col2im, softmax or the dtype casts, and the 16-bit rounding of the
// `half` crate only loosely ("parity unpinned" by the reference); those parts are checked against
// independent numpy formulations in tests/test_extras_cpu.py and tests/test_cast_cpu.py.
//
// Accumulation modes (oracle_set_wide):
//   0 = faithful: sums and dot products accumulate in the element type, ascending
//       logical index (one legal schedule of the reference's rayon + Mutex loops);
//   1 = wide: same formulas, bf16/f16 accumulate in f32 and f32 in f64, one final
//       rounding — the comparison target for large 16-bit reductions / matmuls, where
//       the faithful result is itself dominated by accumulated rounding error.
#include <omp.h>

#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <type_traits>
#include <vector>

#include "half_types.h"

using mxo::bf16;
using mxo::f16;
typedef uint8_t u8;
typedef uint16_t u16;
typedef uint32_t u32;
typedef uint64_t u64;
typedef int8_t i8;
typedef int16_t i16;
typedef int32_t i32;
typedef int64_t i64;
typedef float f32;
typedef double f64;

static int g_wide = 0;
static int g_reduce_parallel = 0;

extern "C" void oracle_set_wide(int wide) { g_wide = wide; }
extern "C" void oracle_set_reduce_parallel(int on) { g_reduce_parallel = on; }
extern "C" void oracle_set_num_threads(int n) { omp_set_num_threads(n > 0 ? n : 1); }
extern "C" int oracle_get_max_threads() { return omp_get_max_threads(); }

// ---------------------------------------------------------------------------------
// type helpers
// ---------------------------------------------------------------------------------
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

template <class T>
static inline T zero_of() {
    if constexpr (is_half_v<T>) return T::from_f32(0.0f);
    else return (T)0;
}

// Rust `as` from float to integer: saturating, NaN -> 0.
template <class T, class F>
static inline T sat_cast(F v) {
    if (v != v) return (T)0;
    const F lo = (F)std::numeric_limits<T>::min();
    // 2^bits as a float is exactly representable; max() itself may round up.
    const F hi_excl = std::is_signed<T>::value ? std::ldexp((F)1, (int)sizeof(T) * 8 - 1) : std::ldexp((F)1, (int)sizeof(T) * 8);
    if (v <= lo) return std::numeric_limits<T>::min();
    if (v >= hi_excl) return std::numeric_limits<T>::max();
    return (T)v;
}

template <class T>
static inline T wrap_add(T a, T b) {
    typedef typename std::make_unsigned<T>::type U;
    return (T)(U)((U)a + (U)b);
}
template <class T>
static inline T wrap_mul(T a, T b) {
    // promote to 64-bit unsigned to avoid int-promotion overflow UB on u16
    return (T)(u64)((u64)(typename std::make_unsigned<T>::type)a * (u64)(typename std::make_unsigned<T>::type)b);
}
template <class T>
static inline T wrap_neg(T a) {
    typedef typename std::make_unsigned<T>::type U;
    return (T)(U)((U)0 - (U)a);
}
template <class T>
static inline T wrap_abs(T a) {
    return a < 0 ? wrap_neg(a) : a;
}
template <class T>
static inline T sat_add(T a, T b) {
    T r;
    if (!__builtin_add_overflow(a, b, &r)) return r;
    if (std::is_signed<T>::value) return a < 0 ? std::numeric_limits<T>::min() : std::numeric_limits<T>::max();
    return std::numeric_limits<T>::max();
}
template <class T>
static inline T sat_sub(T a, T b) {
    T r;
    if (!__builtin_sub_overflow(a, b, &r)) return r;
    if (std::is_signed<T>::value) return a < 0 ? std::numeric_limits<T>::min() : std::numeric_limits<T>::max();
    return std::numeric_limits<T>::min();
}
template <class T>
static inline T sat_mul(T a, T b) {
    T r;
    if (!__builtin_mul_overflow(a, b, &r)) return r;
    if (std::is_signed<T>::value) return ((a < 0) != (b < 0)) ? std::numeric_limits<T>::min() : std::numeric_limits<T>::max();
    return std::numeric_limits<T>::max();
}
template <class T>
static inline T sat_div(T a, T b) {  // b != 0
    if (std::is_signed<T>::value && a == std::numeric_limits<T>::min() && b == (T)-1) return std::numeric_limits<T>::max();
    return (T)(a / b);
}

// ---------------------------------------------------------------------------------
// layout helpers — crates/maidenx_cpu/src/utils.rs
// ---------------------------------------------------------------------------------
static inline bool is_contiguous(size_t num_dims, const size_t* dims, const size_t* strides) {  // utils.rs:2-12
    size_t acc = 1;
    for (size_t d = 0; d < num_dims; d++) {
        size_t k = num_dims - 1 - d;
        if (dims[k] > 1 && acc != strides[k]) return false;
        acc *= dims[k];
    }
    return true;
}
static inline size_t get_strided_index(size_t idx, size_t num_dims, const size_t* dims, const size_t* strides) {  // utils.rs:15-31
    size_t s = 0, rem = idx;
    for (size_t d = 0; d < num_dims; d++) {
        size_t k = num_dims - 1 - d;
        if (strides[k] != 0) s += (rem % dims[k]) * strides[k];
        rem /= dims[k];
    }
    return s;
}

// ---------------------------------------------------------------------------------
// binary lambdas — crates/maidenx_cpu/src/ops/binary.rs:372-606
// ---------------------------------------------------------------------------------
struct BAdd {
    template <class T>
    static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a | b;
        else if constexpr (is_int_v<T>) return sat_add(a, b);
        else return a + b;
    }
};
struct BSub {
    template <class T>
    static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & b;
        else if constexpr (is_int_v<T>) return sat_sub(a, b);
        else return a - b;
    }
};
struct BMul {
    template <class T>
    static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a ^ b;
        else if constexpr (is_int_v<T>) return sat_mul(a, b);
        else return a * b;
    }
};
struct BDiv {  // binary.rs:414-578: x/0 -> 0 when x == 0, else +inf (floats) / MAX or MIN by sign (ints)
    template <class T>
    static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & b;
        else if constexpr (is_int_v<T>) {
            if (b == 0) {
                if (a == 0) return 0;
                if (std::is_signed<T>::value && a < 0) return std::numeric_limits<T>::min();
                return std::numeric_limits<T>::max();
            }
            return sat_div(a, b);
        } else if constexpr (is_half_v<T>) {
            if (b == zero_of<T>()) return a == zero_of<T>() ? zero_of<T>() : T::from_f32(INFINITY);
            return a / b;
        } else {
            if (b == (T)0) return a == (T)0 ? (T)0 : (T)INFINITY;
            return a / b;
        }
    }
};
struct BMax {  // binary.rs:580-592: f32/f64 use Rust `max` (NaN-ignoring), 16-bit use `a > b ? a : b`
    template <class T>
    static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a | b;
        else if constexpr (is_fp_v<T>) return std::fmax(a, b);
        else return a > b ? a : b;
    }
};
struct BMin {
    template <class T>
    static T f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & b;
        else if constexpr (is_fp_v<T>) return std::fmin(a, b);
        else return a < b ? a : b;
    }
};
struct BEq {
    template <class T>
    static bool f(T a, T b) { return a == b; }
};
struct BNe {
    template <class T>
    static bool f(T a, T b) { return a != b; }
};
struct BLt {
    template <class T>
    static bool f(T a, T b) {
        if constexpr (is_bool_v<T>) return !a & b;
        else return a < b;
    }
};
struct BLe {
    template <class T>
    static bool f(T a, T b) { return a <= b; }
};
struct BGt {
    template <class T>
    static bool f(T a, T b) {
        if constexpr (is_bool_v<T>) return a & !b;
        else return a > b;
    }
};
struct BGe {
    template <class T>
    static bool f(T a, T b) { return a >= b; }
};
template <class T>
static inline bool truthy(T a) {
    return a != zero_of<T>();
}
struct BLAnd {
    template <class T>
    static bool f(T a, T b) { return truthy(a) && truthy(b); }
};
struct BLOr {
    template <class T>
    static bool f(T a, T b) { return truthy(a) || truthy(b); }
};
struct BLXor {
    template <class T>
    static bool f(T a, T b) { return truthy(a) != truthy(b); }
};

// binary.rs:13-124 (and the logical_op twin :250-370): out is contiguous from 0;
// operand index = sum of coord*stride over dims (the stride-0 test in the reference
// is a no-op for the value).
template <class Op, class T, class O>
static void binary_driver(size_t num_els, size_t num_dims, const size_t* meta, const T* lhs, const T* rhs, O* out) {
    const size_t* dims = meta;
    const size_t* ls = meta ? meta + num_dims : nullptr;
    const size_t* rs = meta ? meta + 2 * num_dims : nullptr;
    size_t lo = meta ? meta[3 * num_dims] : 0, ro = meta ? meta[3 * num_dims + 1] : 0;
    bool lc = meta ? is_contiguous(num_dims, dims, ls) : true;
    bool rc = meta ? is_contiguous(num_dims, dims, rs) : true;
    lhs += lo;
    rhs += ro;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < num_els; i++) {
        size_t li = i, ri = i;
        if (!lc || !rc) {
            size_t tmp = i, a = 0, b = 0;
            for (size_t dd = num_dims; dd-- > 0;) {
                size_t c = tmp % dims[dd];
                a += c * ls[dd];
                b += c * rs[dd];
                tmp /= dims[dd];
            }
            if (!lc) li = a;
            if (!rc) ri = b;
        }
        out[i] = (O)Op::template f<T>(lhs[li], rhs[ri]);
    }
}

// binary.rs:126-248: serial in the reference; result written through the lhs index.
template <class Op, class T>
static void binary_inplace_driver(size_t num_els, size_t num_dims, const size_t* meta, T* lhs, const T* rhs) {
    const size_t* dims = meta;
    const size_t* ls = meta ? meta + num_dims : nullptr;
    const size_t* rs = meta ? meta + 2 * num_dims : nullptr;
    size_t lo = meta ? meta[3 * num_dims] : 0, ro = meta ? meta[3 * num_dims + 1] : 0;
    size_t nd = meta ? num_dims : 0;
    bool lc = is_contiguous(nd, dims, ls);
    bool rc = is_contiguous(nd, dims, rs);
    for (size_t i = 0; i < num_els; i++) {
        size_t li = i, ri = i;
        if (!lc || !rc) {
            size_t tmp = i, a = 0, b = 0;
            for (size_t dd = nd; dd-- > 0;) {
                size_t c = tmp % dims[dd];
                a += c * ls[dd];
                b += c * rs[dd];
                tmp /= dims[dd];
            }
            if (!lc) li = a;
            if (!rc) ri = b;
        }
        T* p = lhs + lo + li;
        *p = Op::template f<T>(*p, rhs[ro + ri]);
    }
}

// ---------------------------------------------------------------------------------
// unary lambdas — crates/maidenx_cpu/src/ops/unary.rs:124-741
// 16-bit floats: computed in f32 and rounded once (unary.rs:141-142, 279-293).
// ---------------------------------------------------------------------------------
template <class T, class F32Fn, class F64Fn>
static inline T fp_apply(T x, F32Fn f32fn, F64Fn f64fn) {
    if constexpr (is_half_v<T>) return T::from_f32(f32fn(x.to_f32()));
    else if constexpr (std::is_same<T, f32>::value) return f32fn(x);
    else return f64fn(x);
}
#define FP_UNARY(NAME, EXPR32, EXPR64)                                                            \
    struct NAME {                                                                                 \
        template <class T>                                                                        \
        static T f(T x) {                                                                         \
            if constexpr (is_bool_v<T>) return x;                                                 \
            else return fp_apply(x, [](f32 v) -> f32 { return EXPR32; }, [](f64 v) -> f64 { return EXPR64; }); \
        }                                                                                         \
    };
FP_UNARY(USigmoid, 1.0f / (1.0f + std::exp(-v)), 1.0 / (1.0 + std::exp(-v)))
FP_UNARY(UTanh, std::tanh(v), std::tanh(v))
FP_UNARY(USin, std::sin(v), std::sin(v))
FP_UNARY(UCos, std::cos(v), std::cos(v))
FP_UNARY(UTan, std::tan(v), std::tan(v))
FP_UNARY(ULn, std::log(v), std::log(v))
FP_UNARY(ULog10, std::log10(v), std::log10(v))
FP_UNARY(ULog2, std::log2(v), std::log2(v))
FP_UNARY(UExp, std::exp(v), std::exp(v))
FP_UNARY(UExp10, std::pow(10.0f, v), std::pow(10.0, v))  // unary.rs:333: 10f32.powf(x)
FP_UNARY(UExp2, std::exp2(v), std::exp2(v))
FP_UNARY(USoftplus, std::log(1.0f + std::exp(v)), std::log(1.0 + std::exp(v)))
FP_UNARY(URecip, 1.0f / v, 1.0 / v)
#undef FP_UNARY

static inline f32 gelu32(f32 x) {  // unary.rs:268-273
    const f32 s = 0.7978845608028654f, c = 0.044715f;
    f32 t = s * (x + c * x * x * x);
    return 0.5f * x * (1.0f + std::tanh(t));
}
static inline f64 gelu64(f64 x) {
    const f64 s = 0.7978845608028654, c = 0.044715;
    f64 t = s * (x + c * x * x * x);
    return 0.5 * x * (1.0 + std::tanh(t));
}
struct UGelu {
    template <class T>
    static T f(T x) { return fp_apply(x, gelu32, gelu64); }
};
struct UNeg {
    template <class T>
    static T f(T x) {
        if constexpr (is_bool_v<T>) return !x;
        else if constexpr (is_int_v<T>) return wrap_neg(x);
        else return -x;
    }
};
struct UAbs {
    template <class T>
    static T f(T x) {
        if constexpr (is_bool_v<T>) return x;
        else if constexpr (is_int_v<T>) return wrap_abs(x);
        else if constexpr (is_half_v<T>) return T::from_f32(std::fabs(x.to_f32()));
        else return std::fabs(x);
    }
};
struct USign {
    template <class T>
    static T f(T x) {
        if constexpr (is_bool_v<T>) return x;
        else if constexpr (is_half_v<T>) {
            T z = zero_of<T>();
            return x > z ? T::from_f32(1.0f) : (x < z ? T::from_f32(-1.0f) : z);
        } else if constexpr (std::is_unsigned<T>::value) return x > 0 ? 1 : 0;
        else return x > 0 ? (T)1 : (x < 0 ? (T)-1 : (T)0);
    }
};
struct USquare {
    template <class T>
    static T f(T x) {
        if constexpr (is_bool_v<T>) return x;
        else if constexpr (is_int_v<T>) return wrap_mul(x, x);
        else return x * x;
    }
};
struct USqrt {  // unary.rs:219-232: integers go through f32 (i64 through f64) of |x|, truncating
    template <class T>
    static T f(T x) {
        if constexpr (is_bool_v<T>) return x;
        else if constexpr (is_half_v<T>) return T::from_f32(std::sqrt(x.to_f32()));
        else if constexpr (is_fp_v<T>) return std::sqrt(x);
        else if constexpr (std::is_same<T, i64>::value) return sat_cast<T, f64>(std::sqrt((f64)wrap_abs(x)));
        else if constexpr (std::is_signed<T>::value) return sat_cast<T, f32>(std::sqrt((f32)wrap_abs(x)));
        else return sat_cast<T, f32>(std::sqrt((f32)x));
    }
};
struct URelu {
    template <class T>
    static T f(T x) {
        if constexpr (is_bool_v<T>) return x;
        else return x > zero_of<T>() ? x : zero_of<T>();
    }
};
struct ULogicalNot {
    template <class T>
    static bool f(T x) {
        if constexpr (is_bool_v<T>) return !x;
        else return x == zero_of<T>();
    }
};

// with constant — unary.rs:374-741
struct CAdd {
    template <class T>
    static T f(T x, T c) { return BAdd::f<T>(x, c); }
};
struct CSub {
    template <class T>
    static T f(T x, T c) { return BSub::f<T>(x, c); }
};
struct CMul {
    template <class T>
    static T f(T x, T c) { return BMul::f<T>(x, c); }
};
struct CDiv {
    template <class T>
    static T f(T x, T c) { return BDiv::f<T>(x, c); }
};
struct CMax {
    template <class T>
    static T f(T x, T c) { return BMax::f<T>(x, c); }
};
struct CMin {
    template <class T>
    static T f(T x, T c) { return BMin::f<T>(x, c); }
};
struct CPow {  // unary.rs:562-578
    template <class T>
    static T f(T x, T c) {
        if constexpr (is_bool_v<T>) return x;
        else if constexpr (is_half_v<T>) return T::from_f32(std::pow(x.to_f32(), c.to_f32()));
        else if constexpr (is_fp_v<T>) return std::pow(x, c);
        else if constexpr (std::is_same<T, u8>::value) return sat_cast<T, f32>(std::pow((f32)x, (f32)c));
        else return sat_cast<T, f64>(std::pow((f64)x, (f64)c));
    }
};
struct CLeakyRelu {
    template <class T>
    static T f(T x, T a) { return x > zero_of<T>() ? x : a * x; }
};
struct CElu {  // unary.rs:601-636
    template <class T>
    static T f(T x, T a) {
        if constexpr (is_half_v<T>) {
            f32 xf = x.to_f32(), af = a.to_f32();
            return xf > 0.0f ? x : T::from_f32(af * (std::exp(xf) - 1.0f));
        } else return x > (T)0 ? x : a * (std::exp(x) - (T)1);
    }
};
struct CEq {
    template <class T>
    static bool f(T x, T c) { return x == c; }
};
struct CNe {
    template <class T>
    static bool f(T x, T c) { return x != c; }
};
struct CLt {
    template <class T>
    static bool f(T x, T c) {
        if constexpr (is_bool_v<T>) return (!x) && c;
        else return x < c;
    }
};
struct CLe {
    template <class T>
    static bool f(T x, T c) {
        if constexpr (is_bool_v<T>) return (!x) || c;
        else return x <= c;
    }
};
struct CGt {
    template <class T>
    static bool f(T x, T c) {
        if constexpr (is_bool_v<T>) return x && (!c);
        else return x > c;
    }
};
struct CGe {
    template <class T>
    static bool f(T x, T c) {
        if constexpr (is_bool_v<T>) return x || (!c);
        else return x >= c;
    }
};

// unary.rs:14-62 / :71-122
template <class Op, class T, class O>
static void unary_driver(size_t num_els, size_t num_dims, const size_t* meta, const T* in, O* out) {
    const size_t* dims = meta;
    const size_t* st = meta ? meta + num_dims : nullptr;
    size_t off = meta ? meta[2 * num_dims] : 0;
    bool cont = meta ? is_contiguous(num_dims, dims, st) : true;
    in += off;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < num_els; i++) {
        size_t si = cont ? i : get_strided_index(i, num_dims, dims, st);
        out[i] = (O)Op::template f<T>(in[si]);
    }
}
template <class Op, class T, class O>
static void unary_const_driver(size_t num_els, size_t num_dims, const size_t* meta, const T* in, T c, O* out) {
    const size_t* dims = meta;
    const size_t* st = meta ? meta + num_dims : nullptr;
    size_t off = meta ? meta[2 * num_dims] : 0;
    bool cont = meta ? is_contiguous(num_dims, dims, st) : true;
    in += off;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < num_els; i++) {
        size_t si = cont ? i : get_strided_index(i, num_dims, dims, st);
        out[i] = (O)Op::template f<T>(in[si], c);
    }
}

// ---------------------------------------------------------------------------------
// reductions — crates/maidenx_cpu/src/ops/reduction.rs
// ---------------------------------------------------------------------------------
template <class T>
struct WideAcc {
    typedef T type;
};
template <>
struct WideAcc<bf16> {
    typedef f32 type;
};
template <>
struct WideAcc<f16> {
    typedef f32 type;
};
template <>
struct WideAcc<f32> {
    typedef f64 type;
};

template <class A, class T>
static inline A to_acc(T v) {
    if constexpr (is_half_v<T> && !is_half_v<A>) return (A)v.to_f32();
    else return (A)v;
}
template <class T, class A>
static inline T from_acc(A a) {
    if constexpr (is_half_v<T> && !is_half_v<A>) return T::from_f32((f32)a);
    else return (T)a;
}
template <class A>
static inline void acc_add(A& a, A v) {
    if constexpr (std::is_integral<A>::value) a = wrap_add(a, v);
    else a += v;
}

enum { R_SUM = 0, R_MEAN = 1, R_MAX = 2, R_MIN = 3 };

struct SpinLocks {
    std::vector<std::atomic_flag> f;
    explicit SpinLocks(size_t n) : f(n) {
        for (auto& x : f) x.clear();
    }
    void lock(size_t i) {
        while (f[i].test_and_set(std::memory_order_acquire)) {
        }
    }
    void unlock(size_t i) { f[i].clear(std::memory_order_release); }
};

// reduction.rs:45-58 (contiguous) / :60-79 (strided): fold the logical index over each reduced dim.
static inline size_t fold_dst(size_t i, size_t nr, const size_t* rl, const size_t* rs, bool cont) {
    size_t dst = i;
    for (size_t nd = 0; nd < nr; nd++) {
        size_t s = rs[nd];
        if (cont || s != 0) {
            size_t pre = dst / s, post = dst % s;
            dst = (pre / rl[nd]) * s + post;
        } else {
            dst /= rl[nd];
        }
    }
    return dst;
}

template <class T, int KIND, class A>
static void reduce_impl(size_t num_els, size_t num_dims, size_t nr, const size_t* meta, const T* inp, T* out) {
    const size_t* dims = meta;
    const size_t* st = meta + num_dims;
    const size_t* rl = meta + 2 * num_dims;
    const size_t* rs = meta + 2 * num_dims + nr;
    size_t off = meta[2 * num_dims + 2 * nr];
    inp += off;
    size_t out_size = num_els, factor = 1;
    for (size_t i = 0; i < nr; i++) {
        out_size /= rl[i];
        factor *= rl[i];
    }
    bool cont = is_contiguous(num_dims, dims, st);
    A init;
    if constexpr (KIND == R_MAX) {  // reduction.rs:603-614: floats start from f32::MIN / f64::MIN (16-bit: rounds to -inf)
        if constexpr (is_half_v<T>) init = to_acc<A>(T::from_f32(-std::numeric_limits<f32>::max()));
        else if constexpr (is_fp_v<T>) init = (A)-std::numeric_limits<T>::max();
        else init = (A)std::numeric_limits<T>::min();
    } else if constexpr (KIND == R_MIN) {
        if constexpr (is_half_v<T>) init = to_acc<A>(T::from_f32(std::numeric_limits<f32>::max()));
        else if constexpr (is_fp_v<T>) init = (A)std::numeric_limits<T>::max();
        else init = (A)std::numeric_limits<T>::max();
    } else {
        init = to_acc<A>(zero_of<T>());
    }
    std::vector<A> acc(out_size, init);
    auto body = [&](size_t i) {
        size_t src = cont ? i : get_strided_index(i, num_dims, dims, st);
        size_t dst = fold_dst(i, nr, rl, rs, cont);
        A v = to_acc<A>(inp[src]);
        return std::pair<size_t, A>(dst, v);
    };
    auto combine = [&](A& a, A v) {
        if constexpr (KIND == R_MAX) a = (v > a) ? v : a;  // reduction.rs:432-434
        else if constexpr (KIND == R_MIN) a = (v < a) ? v : a;
        else acc_add(a, v);
    };
    if (g_reduce_parallel && omp_get_max_threads() > 1) {
        SpinLocks locks(out_size);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < num_els; i++) {
            auto p = body(i);
            locks.lock(p.first);
            combine(acc[p.first], p.second);
            locks.unlock(p.first);
        }
    } else {
        for (size_t i = 0; i < num_els; i++) {
            auto p = body(i);
            combine(acc[p.first], p.second);
        }
    }
    for (size_t j = 0; j < out_size; j++) {
        if constexpr (KIND == R_MEAN) {  // reduction.rs:263-268: finished sum / factor, in the element type
            if constexpr (is_half_v<T>) {
                if constexpr (is_half_v<A>) out[j] = acc[j] / T::from_f32((f32)factor);
                else out[j] = T::from_f32(acc[j] / T::from_f32((f32)factor).to_f32());
            } else out[j] = (T)(acc[j] / (A)(T)factor);
        } else out[j] = from_acc<T>(acc[j]);
    }
}
template <class T, int KIND>
static void reduce_op(size_t num_els, size_t num_dims, size_t nr, const size_t* meta, const T* inp, T* out) {
    typedef typename WideAcc<T>::type W;
    if (g_wide && !std::is_same<W, T>::value && (KIND == R_SUM || KIND == R_MEAN)) reduce_impl<T, KIND, W>(num_els, num_dims, nr, meta, inp, out);
    else reduce_impl<T, KIND, T>(num_els, num_dims, nr, meta, inp, out);
}

// reduction.rs:91-183
template <class T, class A>
static void sum_to_shape_impl(size_t num_els, size_t num_dims, const size_t* meta, const T* inp, T* out) {
    const size_t* idims = meta;
    const size_t* ist = meta + num_dims;
    const size_t* odims = meta + 2 * num_dims;
    size_t off = meta[3 * num_dims];
    const T* input = inp + off;
    size_t out_size = 1;
    for (size_t d = 0; d < num_dims; d++) out_size *= odims[d];
    std::vector<size_t> rf(num_dims);
    for (size_t d = 0; d < num_dims; d++) rf[d] = idims[d] / odims[d];
    bool cont = is_contiguous(num_dims, idims, ist);
    std::vector<A> acc(out_size, to_acc<A>(zero_of<T>()));
    auto body = [&](size_t i) {
        size_t coords[32];
        size_t tmp = i;
        for (size_t d = num_dims; d-- > 0;) {
            coords[d] = tmp % idims[d];
            tmp /= idims[d];
        }
        size_t dst = 0;
        for (size_t d = 0; d < num_dims; d++) dst = dst * odims[d] + coords[d] / rf[d];
        size_t src = i;
        if (!cont) {  // reduction.rs:157-166: the offset is applied twice and wrapped by num_els
            size_t s = 0;
            for (size_t d = 0; d < num_dims; d++) s += coords[d] * ist[d];
            src = (s + off) % num_els;
        }
        return std::pair<size_t, A>(dst, to_acc<A>(input[src]));
    };
    if (g_reduce_parallel && omp_get_max_threads() > 1) {
        SpinLocks locks(out_size);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < num_els; i++) {
            auto p = body(i);
            locks.lock(p.first);
            acc_add(acc[p.first], p.second);
            locks.unlock(p.first);
        }
    } else {
        for (size_t i = 0; i < num_els; i++) {
            auto p = body(i);
            acc_add(acc[p.first], p.second);
        }
    }
    for (size_t j = 0; j < out_size; j++) out[j] = from_acc<T>(acc[j]);
}
template <class T>
static void sum_to_shape_op(size_t num_els, size_t num_dims, const size_t* meta, const T* inp, T* out) {
    typedef typename WideAcc<T>::type W;
    if (g_wide && !std::is_same<W, T>::value) sum_to_shape_impl<T, W>(num_els, num_dims, meta, inp, out);
    else sum_to_shape_impl<T, T>(num_els, num_dims, meta, inp, out);
}

// ---------------------------------------------------------------------------------
// matmul — crates/maidenx_cpu/src/ops/matmul.rs
// ---------------------------------------------------------------------------------
template <class T, class A>
static inline void mac(A& acc, T a, T b) {
    if constexpr (std::is_integral<T>::value) acc = wrap_add<A>(acc, wrap_mul<T>(a, b));
    else if constexpr (std::is_same<A, T>::value) acc += a * b;  // product and sum each rounded to T
    else acc += to_acc<A>(a) * to_acc<A>(b);
}

template <class T, class A>
static void matmul_impl(size_t num_els, const size_t* meta, const T* a, const T* b, T* c) {  // matmul.rs:19-120
    if (!meta || !a || !b || !c) return;
    size_t out_nd = meta[0], a_nd = meta[1], b_nd = meta[2];
    if (a_nd == 0 || b_nd == 0) return;
    const size_t* out_shape = meta + 3;
    const size_t* a_shape = out_shape + out_nd;
    const size_t* b_shape = a_shape + a_nd;
    const size_t* a_st = b_shape + b_nd;
    const size_t* b_st = a_st + a_nd;
    size_t a_off = b_st[b_nd], b_off = b_st[b_nd + 1];
    size_t m = out_nd >= 2 ? out_shape[out_nd - 2] : 1;
    size_t n = out_nd >= 1 ? out_shape[out_nd - 1] : 1;
    size_t k = a_shape[a_nd - 1];
    if (m == 0 || n == 0 || k == 0) return;
    bool ac = is_contiguous(a_nd, a_shape, a_st), bc = is_contiguous(b_nd, b_shape, b_st);
    size_t a_size = num_els * k, b_size = num_els * k;
    a += a_off;
    b += b_off;
    size_t rows = (num_els + n - 1) / n;
#pragma omp parallel for schedule(static)
    for (size_t bm = 0; bm < rows; bm++) {
        size_t batch = bm / m, mi = bm % m;
        size_t row_len = (bm + 1) * n <= num_els ? n : num_els - bm * n;
        for (size_t ni = 0; ni < n; ni++) {
            A acc = to_acc<A>(zero_of<T>());
            if (ac && bc) {
                size_t ab = batch * (m * k) + mi * k, bb = batch * (k * n);
                for (size_t ki = 0; ki < k; ki++) {
                    size_t ai = ab + ki, bi = bb + ki * n + ni;
                    if (ai < a_size && bi < b_size) mac<T, A>(acc, a[ai], b[bi]);
                }
            } else {
                for (size_t ki = 0; ki < k; ki++) {
                    size_t ai = a_nd >= 2 ? batch * a_st[0] + mi * a_st[a_nd - 2] + ki * a_st[a_nd - 1] : ki * a_st[0];
                    size_t bi = b_nd >= 2 ? batch * b_st[0] + ki * b_st[b_nd - 2] + ni * b_st[b_nd - 1] : ni * b_st[0];
                    if (ai < a_size && bi < b_size) mac<T, A>(acc, a[ai], b[bi]);
                }
            }
            if (ni < row_len) c[bm * n + ni] = from_acc<T>(acc);
        }
    }
}
template <class T>
static void matmul_op(size_t num_els, const size_t* meta, const T* a, const T* b, T* c) {
    typedef typename WideAcc<T>::type W;
    if (g_wide && !std::is_same<W, T>::value) matmul_impl<T, W>(num_els, meta, a, b, c);
    else matmul_impl<T, T>(num_els, meta, a, b, c);
}

template <class T, class A>
static void matmul_backward_impl(size_t nea, size_t neb, const size_t* meta, const T* g, const T* a, const T* b, T* ga, T* gb) {  // matmul.rs:137-266
    if (!meta || !g || !a || !b) return;
    size_t out_nd = meta[0], a_nd = meta[1], b_nd = meta[2];
    if (a_nd == 0 || b_nd == 0) return;
    const size_t* out_shape = meta + 3;
    const size_t* a_shape = out_shape + out_nd;
    const size_t* b_shape = a_shape + a_nd;
    const size_t* tail = b_shape + b_nd + a_nd + b_nd;
    size_t a_off = tail[0], b_off = tail[1];
    size_t m = out_nd >= 2 ? out_shape[out_nd - 2] : 1;
    size_t n = out_nd >= 1 ? out_shape[out_nd - 1] : 1;
    size_t k = b_nd >= 2 ? b_shape[b_nd - 2] : a_shape[a_nd - 1];
    if (m == 0 || n == 0 || k == 0) return;
    size_t gsize = 1;
    for (size_t d = 0; d < out_nd; d++) gsize *= out_shape[d];
    if (gsize == 0) return;
    if (ga) {
        const T* bs = b + b_off;
        size_t rows = (nea + k - 1) / k;
#pragma omp parallel for schedule(static)
        for (size_t bm = 0; bm < rows; bm++) {
            size_t batch = bm / m, mi = bm % m;
            size_t row_len = (bm + 1) * k <= nea ? k : nea - bm * k;
            for (size_t ki = 0; ki < k; ki++) {
                A acc = to_acc<A>(zero_of<T>());
                if (out_nd == 0) {
                    if (ki < neb) {
                        if constexpr (std::is_integral<T>::value) acc = (A)wrap_mul<T>(g[0], bs[ki]);
                        else if constexpr (std::is_same<A, T>::value) acc = g[0] * bs[ki];
                        else acc = to_acc<A>(g[0]) * to_acc<A>(bs[ki]);
                    }
                } else {
                    size_t gbase = batch * (m * n) + mi * n, bbase = batch * (k * n);
                    for (size_t ni = 0; ni < n; ni++)
                        if (gbase + ni < gsize && bbase + ki * n + ni < neb) mac<T, A>(acc, g[gbase + ni], bs[bbase + ki * n + ni]);
                }
                if (ki < row_len) ga[bm * k + ki] = from_acc<T>(acc);
            }
        }
    }
    if (gb) {
        const T* as = a + a_off;
        size_t rows = (neb + n - 1) / n;
#pragma omp parallel for schedule(static)
        for (size_t bk = 0; bk < rows; bk++) {
            size_t batch = bk / k, ki = bk % k;
            size_t row_len = (bk + 1) * n <= neb ? n : neb - bk * n;
            for (size_t ni = 0; ni < n; ni++) {
                A acc = to_acc<A>(zero_of<T>());
                if (out_nd == 0) {
                    if (ki < nea) {
                        if constexpr (std::is_integral<T>::value) acc = (A)wrap_mul<T>(g[0], as[ki]);
                        else if constexpr (std::is_same<A, T>::value) acc = g[0] * as[ki];
                        else acc = to_acc<A>(g[0]) * to_acc<A>(as[ki]);
                    }
                } else {
                    size_t abase = batch * (m * k), gbase = batch * (m * n);
                    for (size_t mi = 0; mi < m; mi++) {
                        size_t ai = abase + mi * k + ki, gi = gbase + mi * n + ni;
                        if (ai < nea && gi < gsize) mac<T, A>(acc, as[ai], g[gi]);
                    }
                }
                if (ni < row_len) gb[bk * n + ni] = from_acc<T>(acc);
            }
        }
    }
}
template <class T>
static void matmul_backward_op(size_t nea, size_t neb, const size_t* meta, const T* g, const T* a, const T* b, T* ga, T* gb) {
    typedef typename WideAcc<T>::type W;
    if (g_wide && !std::is_same<W, T>::value) matmul_backward_impl<T, W>(nea, neb, meta, g, a, b, ga, gb);
    else matmul_backward_impl<T, T>(nea, neb, meta, g, a, b, ga, gb);
}

// ---------------------------------------------------------------------------------
// conv2d — crates/maidenx_cpu/src/nn/conv.rs
// ---------------------------------------------------------------------------------
template <class T>
static void im2col_op(size_t num_els, const size_t* md, const T* input, T* col) {  // conv.rs:23-72
    if (!md || !input || !col) return;
    size_t B = md[0], C = md[1], H = md[2], W = md[3], KH = md[4], KW = md[5], OH = md[6], OW = md[7];
    size_t PH = md[8], PW = md[9], SH = md[10], SW = md[11];
    size_t ksz = KH * KW, osz = OH * OW, chunk = C * ksz * osz;
    if (chunk == 0) return;
    size_t nb = (num_els + chunk - 1) / chunk;
    (void)B;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < nb; b++) {
        T* cc = col + b * chunk;
        size_t limit = (b + 1) * chunk <= num_els ? chunk : num_els - b * chunk;
        for (size_t c = 0; c < C; c++)
            for (size_t kh = 0; kh < KH; kh++)
                for (size_t kw = 0; kw < KW; kw++) {
                    size_t ioff = b * C * H * W + c * H * W;
                    size_t coff = (c * ksz + kh * KW + kw) * osz;
                    for (size_t ho = 0; ho < OH; ho++) {
                        ptrdiff_t hi = (ptrdiff_t)(ho * SH) - (ptrdiff_t)PH + (ptrdiff_t)kh;
                        for (size_t wo = 0; wo < OW; wo++) {
                            ptrdiff_t wi = (ptrdiff_t)(wo * SW) - (ptrdiff_t)PW + (ptrdiff_t)kw;
                            size_t ci = coff + ho * OW + wo;
                            if (ci >= limit) continue;
                            bool in = hi >= 0 && hi < (ptrdiff_t)H && wi >= 0 && wi < (ptrdiff_t)W;
                            cc[ci] = in ? input[ioff + (size_t)hi * W + (size_t)wi] : zero_of<T>();
                        }
                    }
                }
    }
}
template <class T>
static void col2im_op(size_t num_els, const size_t* md, const T* col, T* output) {  // conv.rs:94-148
    if (!md || !col || !output) return;
    size_t B = md[0], C = md[1], H = md[2], W = md[3], KH = md[4], KW = md[5], OH = md[6], OW = md[7];
    size_t PH = md[8], PW = md[9], SH = md[10], SW = md[11];
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < B; b++) {
        T* oc = output + b * C * H * W;
        for (size_t c = 0; c < C; c++)
            for (size_t h = 0; h < H; h++) {
                size_t hp = h + PH;
                for (size_t w = 0; w < W; w++) {
                    size_t wp = w + PW;
                    size_t hs0 = hp >= KH - 1 ? hp - (KH - 1) : 0, ws0 = wp >= KW - 1 ? wp - (KW - 1) : 0;
                    size_t hs = (hs0 + SH - 1) / SH, ws = (ws0 + SW - 1) / SW;
                    size_t he = hp / SH + 1 < OH ? hp / SH + 1 : OH;
                    size_t we = wp / SW + 1 < OW ? wp / SW + 1 : OW;
                    T sum = zero_of<T>();
                    for (size_t ho = hs; ho < he; ho++)
                        for (size_t wo = ws; wo < we; wo++) {
                            size_t kh = hp - ho * SH, kw = wp - wo * SW;
                            if (kh < KH && kw < KW) {
                                size_t ci = (((b * C + c) * KH * KW + kh * KW + kw) * OH + ho) * OW + wo;
                                if (ci < num_els) sum += col[ci];
                            }
                        }
                    oc[(c * H + h) * W + w] = sum;
                }
            }
    }
}

// ---------------------------------------------------------------------------------
// exports
// ---------------------------------------------------------------------------------
// 16-bit floats cross the C boundary as their bit patterns (the reference's
// half::bf16 / half::f16 are repr(transparent) u16), bool as one byte 0/1.
#define FOR_ARITH12(X, ...) X(bf16, bf16, ##__VA_ARGS__) X(f16, f16, ##__VA_ARGS__) X(f32, f32, ##__VA_ARGS__) X(f64, f64, ##__VA_ARGS__) \
    X(u8, u8, ##__VA_ARGS__) X(u16, u16, ##__VA_ARGS__) X(u32, u32, ##__VA_ARGS__) X(u64, u64, ##__VA_ARGS__)                               \
    X(i8, i8, ##__VA_ARGS__) X(i16, i16, ##__VA_ARGS__) X(i32, i32, ##__VA_ARGS__) X(i64, i64, ##__VA_ARGS__)
#define FOR_ALL13(X, ...) FOR_ARITH12(X, ##__VA_ARGS__) X(bool, bool, ##__VA_ARGS__)
#define FOR_FLOAT4(X, ...) X(bf16, bf16, ##__VA_ARGS__) X(f16, f16, ##__VA_ARGS__) X(f32, f32, ##__VA_ARGS__) X(f64, f64, ##__VA_ARGS__)
#define FOR_SIGNED8(X, ...) FOR_FLOAT4(X, ##__VA_ARGS__) X(i8, i8, ##__VA_ARGS__) X(i16, i16, ##__VA_ARGS__) X(i32, i32, ##__VA_ARGS__) X(i64, i64, ##__VA_ARGS__)

#define DEF_BIN(SUF, T, NAME, OP) \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, const T* l, const T* r, T* o) { binary_driver<OP, T, T>(n, nd, m, l, r, o); }
#define DEF_BINB(SUF, T, NAME, OP) \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, const T* l, const T* r, bool* o) { binary_driver<OP, T, bool>(n, nd, m, l, r, o); }
#define DEF_BINI(SUF, T, NAME, OP) \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, T* l, const T* r) { binary_inplace_driver<OP, T>(n, nd, m, l, r); }
FOR_ALL13(DEF_BIN, add, BAdd)
FOR_ALL13(DEF_BIN, sub, BSub)
FOR_ALL13(DEF_BIN, mul, BMul)
FOR_ALL13(DEF_BIN, div, BDiv)
FOR_ALL13(DEF_BIN, maximum, BMax)
FOR_ALL13(DEF_BIN, minimum, BMin)
FOR_ALL13(DEF_BINB, logical_and, BLAnd)
FOR_ALL13(DEF_BINB, logical_or, BLOr)
FOR_ALL13(DEF_BINB, logical_xor, BLXor)
FOR_ALL13(DEF_BINB, eq, BEq)
FOR_ALL13(DEF_BINB, ne, BNe)
FOR_ALL13(DEF_BINB, lt, BLt)
FOR_ALL13(DEF_BINB, le, BLe)
FOR_ALL13(DEF_BINB, gt, BGt)
FOR_ALL13(DEF_BINB, ge, BGe)
FOR_ALL13(DEF_BINI, add_inplace, BAdd)
FOR_ALL13(DEF_BINI, sub_inplace, BSub)
FOR_ALL13(DEF_BINI, mul_inplace, BMul)
FOR_ALL13(DEF_BINI, div_inplace, BDiv)

#define DEF_UN(SUF, T, NAME, OP) \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, const T* i, T* o) { unary_driver<OP, T, T>(n, nd, m, i, o); }
#define DEF_UNB(SUF, T, NAME, OP) \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, const T* i, bool* o) { unary_driver<OP, T, bool>(n, nd, m, i, o); }
FOR_SIGNED8(DEF_UN, neg, UNeg)
FOR_SIGNED8(DEF_UN, abs, UAbs)
FOR_ARITH12(DEF_UN, sign, USign)
FOR_ARITH12(DEF_UN, square, USquare)
FOR_ARITH12(DEF_UN, sqrt, USqrt)
FOR_FLOAT4(DEF_UN, relu, URelu)
FOR_FLOAT4(DEF_UN, sigmoid, USigmoid)
FOR_FLOAT4(DEF_UN, tanh, UTanh)
FOR_FLOAT4(DEF_UN, gelu, UGelu)
FOR_FLOAT4(DEF_UN, sin, USin)
FOR_FLOAT4(DEF_UN, cos, UCos)
FOR_FLOAT4(DEF_UN, tan, UTan)
FOR_FLOAT4(DEF_UN, ln, ULn)
FOR_FLOAT4(DEF_UN, log10, ULog10)
FOR_FLOAT4(DEF_UN, log2, ULog2)
FOR_FLOAT4(DEF_UN, exp, UExp)
FOR_FLOAT4(DEF_UN, exp10, UExp10)
FOR_FLOAT4(DEF_UN, exp2, UExp2)
FOR_FLOAT4(DEF_UN, softplus, USoftplus)
FOR_FLOAT4(DEF_UN, recip, URecip)
FOR_ALL13(DEF_UNB, logical_not, ULogicalNot)

// by-value constants: 16-bit floats arrive as their u16 bit pattern
template <class T>
struct CArg {
    typedef T type;
    static T get(T v) { return v; }
};
template <>
struct CArg<bf16> {
    typedef uint16_t type;
    static bf16 get(uint16_t v) { return bf16::from_bits(v); }
};
template <>
struct CArg<f16> {
    typedef uint16_t type;
    static f16 get(uint16_t v) { return f16::from_bits(v); }
};
#define DEF_UC(SUF, T, NAME, OP)                                                                                     \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, const T* i, CArg<T>::type c, T* o) {          \
        unary_const_driver<OP, T, T>(n, nd, m, i, CArg<T>::get(c), o);                                               \
    }
#define DEF_UCB(SUF, T, NAME, OP)                                                                                    \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, const size_t* m, const T* i, CArg<T>::type c, bool* o) {       \
        unary_const_driver<OP, T, bool>(n, nd, m, i, CArg<T>::get(c), o);                                            \
    }
FOR_ARITH12(DEF_UC, add_scalar, CAdd)
FOR_ARITH12(DEF_UC, sub_scalar, CSub)
FOR_ARITH12(DEF_UC, mul_scalar, CMul)
FOR_ARITH12(DEF_UC, div_scalar, CDiv)
FOR_ARITH12(DEF_UC, maximum_scalar, CMax)
FOR_ARITH12(DEF_UC, minimum_scalar, CMin)
FOR_ARITH12(DEF_UC, pow, CPow)
FOR_FLOAT4(DEF_UC, leaky_relu, CLeakyRelu)
FOR_FLOAT4(DEF_UC, elu, CElu)
FOR_ALL13(DEF_UCB, eq_scalar, CEq)
FOR_ALL13(DEF_UCB, ne_scalar, CNe)
FOR_ALL13(DEF_UCB, lt_scalar, CLt)
FOR_ALL13(DEF_UCB, le_scalar, CLe)
FOR_ALL13(DEF_UCB, gt_scalar, CGt)
FOR_ALL13(DEF_UCB, ge_scalar, CGe)

#define DEF_RED(SUF, T, NAME, KIND) \
    extern "C" void NAME##_##SUF(size_t n, size_t nd, size_t nr, const size_t* m, const T* i, T* o) { reduce_op<T, KIND>(n, nd, nr, m, i, o); }
#define DEF_STS(SUF, T) \
    extern "C" void sum_to_shape_##SUF(size_t n, size_t nd, const size_t* m, const T* i, T* o) { sum_to_shape_op<T>(n, nd, m, i, o); }
FOR_ARITH12(DEF_RED, sum, R_SUM)
FOR_FLOAT4(DEF_RED, mean, R_MEAN)
FOR_ARITH12(DEF_RED, max, R_MAX)
FOR_ARITH12(DEF_RED, min, R_MIN)
FOR_ARITH12(DEF_STS)

#define DEF_MM(SUF, T)                                                                                                                   \
    extern "C" void matmul_##SUF(size_t n, const size_t* m, const T* a, const T* b, T* c) { matmul_op<T>(n, m, a, b, c); }               \
    extern "C" void matmul_backward_##SUF(size_t na, size_t nb, const size_t* m, const T* g, const T* a, const T* b, T* ga, T* gb) {     \
        matmul_backward_op<T>(na, nb, m, g, a, b, ga, gb);                                                                               \
    }
FOR_ARITH12(DEF_MM)

#define DEF_CONV(SUF, T)                                                                                                   \
    extern "C" void conv2d_im2col_##SUF(size_t n, const size_t* m, const T* i, T* o) { im2col_op<T>(n, m, i, o); }         \
    extern "C" void conv2d_col2im_##SUF(size_t n, const size_t* m, const T* i, T* o) { col2im_op<T>(n, m, i, o); }
FOR_FLOAT4(DEF_CONV)

// ---------------------------------------------------------------------------------
// fold (the backward of unfold): crates/maidenx_cpu/src/ops/reduction.rs:274-381
// metadata: [dims(n) | strides(n) | fold_dim, window_dim, fold_size, step, window_size, offset]
// ---------------------------------------------------------------------------------
template <class T, class A>
static void fold_impl(size_t num_els, size_t num_dims, const size_t* meta, const T* inp, T* out) {
    const size_t* dims = meta;
    const size_t* strides = meta + num_dims;
    const size_t fold_dim = meta[2 * num_dims], window_dim = meta[2 * num_dims + 1], fold_size = meta[2 * num_dims + 2];
    const size_t step = meta[2 * num_dims + 3], offset = meta[2 * num_dims + 5];
    const T* input = inp + offset;
    size_t out_size = 1;  // :310-319
    for (size_t d = 0; d < num_dims; d++) {
        if (d == window_dim) continue;
        out_size *= d == fold_dim ? fold_size : dims[d];
    }
    std::vector<A> acc(out_size, A());
    std::vector<size_t> coords(num_dims ? num_dims : 1);
    for (size_t i = 0; i < num_els; i++) {  // ascending i: one legal schedule of the reference's parallel loop
        size_t r = i;
        for (size_t d = num_dims; d-- > 0;) {  // :323-339 (both branches are the same row-major split)
            coords[d] = r % dims[d];
            r /= dims[d];
        }
        size_t src = 0;
        for (size_t d = 0; d < num_dims; d++) src += coords[d] * strides[d];
        src %= num_els;  // :345
        const size_t orig_pos = coords[fold_dim] * step + coords[window_dim];
        if (orig_pos >= fold_size) continue;
        size_t dst = 0;
        for (size_t d = 0; d < num_dims; d++) {
            if (d == window_dim) continue;
            dst = d == fold_dim ? dst * fold_size + orig_pos : dst * dims[d] + coords[d];
        }
        acc_add(acc[dst], to_acc<A, T>(input[src]));
    }
    for (size_t j = 0; j < out_size; j++) out[j] = from_acc<T, A>(acc[j]);
}
template <class T>
static void fold_op(size_t num_els, size_t num_dims, const size_t* meta, const T* inp, T* out) {
    if (g_wide) fold_impl<T, typename WideAcc<T>::type>(num_els, num_dims, meta, inp, out);
    else fold_impl<T, T>(num_els, num_dims, meta, inp, out);
}
#define DEF_FOLD(SUF, T) \
    extern "C" void fold_##SUF(size_t n, size_t nd, const size_t* m, const T* i, T* o) { fold_op<T>(n, nd, m, i, o); }
FOR_ARITH12(DEF_FOLD)

// ---------------------------------------------------------------------------------
// padding: crates/maidenx_cpu/src/ops/padding.rs
// metadata: [in_dims(n) | in_strides(n) | in_offset | out_dims(n) | (before, after) x n]
// ---------------------------------------------------------------------------------
enum { P_CONSTANT = 0, P_REFLECTION = 1, P_REPLICATION = 2 };

// Input coordinate of output coordinate `oc` along one dim; false = outside (constant padding only).
template <int MODE>
static inline bool pad_source(long long oc, long long pad_before, long long dim_size, size_t* ic) {
    long long pos = oc - pad_before;
    if (MODE == P_CONSTANT) {  // :71-80
        if (pos < 0 || pos >= dim_size) return false;
    } else if (MODE == P_REFLECTION) {  // :178-196; the tensor layer rejects pads >= dim size, the loop is bounded here all the same
        for (int guard = 0; (pos < 0 || pos >= dim_size) && guard < 64; guard++) pos = pos < 0 ? -pos : 2 * dim_size - pos - 2;
        if (pos < 0 || pos >= dim_size) pos = 0;
    } else {  // :289-295
        pos = pos < 0 ? 0 : (pos > dim_size - 1 ? dim_size - 1 : pos);
    }
    *ic = (size_t)pos;
    return true;
}

template <int MODE>
static inline bool pad_in_index(size_t i, size_t nd, const size_t* in_dims, const size_t* in_strides, const size_t* out_dims, const size_t* pads,
                                bool cont, size_t* in_idx) {
    size_t oc[16], ic[16];
    size_t r = i;
    for (size_t d = nd; d-- > 0;) {
        oc[d] = r % out_dims[d];
        r /= out_dims[d];
    }
    for (size_t d = 0; d < nd; d++)
        if (!pad_source<MODE>((long long)oc[d], (long long)pads[2 * d], (long long)in_dims[d], &ic[d])) return false;
    size_t idx = 0;
    if (cont) {  // :84-92
        size_t stride = 1;
        for (size_t d = nd; d-- > 0;) {
            idx += ic[d] * stride;
            stride *= in_dims[d];
        }
    } else {
        for (size_t d = 0; d < nd; d++) idx += ic[d] * in_strides[d];
    }
    *in_idx = idx;
    return true;
}

template <class T, int MODE>
static void pad_forward(size_t num_els_in, size_t num_els_out, size_t nd, const size_t* meta, const T* inp, T* out, T pad_value) {
    (void)num_els_in;
    if (nd > 16) return;
    const size_t* in_dims = meta;
    const size_t* in_strides = meta + nd;
    const size_t in_off = meta[2 * nd];
    const size_t* out_dims = meta + 2 * nd + 1;
    const size_t* pads = meta + 3 * nd + 1;
    const bool cont = is_contiguous(nd, in_dims, in_strides);
    const T* input = inp + in_off;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)num_els_out; i++) {
        size_t idx;
        out[i] = pad_in_index<MODE>((size_t)i, nd, in_dims, in_strides, out_dims, pads, cont, &idx) ? input[idx] : pad_value;
    }
}

// :327-436, :438-558, :560-664: grad_in[in_offset + in_idx] accumulates every grad_out element that maps to it;
// the whole block of num_els_in elements is overwritten (zeros where nothing maps).
template <class T, int MODE, class A>
static void pad_backward_impl(size_t num_els_in, size_t num_els_out, size_t nd, const size_t* meta, const T* grad_out, T* grad_in) {
    if (nd > 16) return;
    const size_t* in_dims = meta;
    const size_t* in_strides = meta + nd;
    const size_t in_off = meta[2 * nd];
    const size_t* out_dims = meta + 2 * nd + 1;
    const size_t* pads = meta + 3 * nd + 1;
    const bool cont = is_contiguous(nd, in_dims, in_strides);
    std::vector<A> acc(num_els_in, A());
    for (size_t i = 0; i < num_els_out; i++) {
        size_t idx;
        if (pad_in_index<MODE>(i, nd, in_dims, in_strides, out_dims, pads, cont, &idx) && idx < num_els_in) acc_add(acc[idx], to_acc<A, T>(grad_out[i]));
    }
    for (size_t j = 0; j < num_els_in; j++) grad_in[in_off + j] = from_acc<T, A>(acc[j]);
}
template <class T, int MODE>
static void pad_backward(size_t ni, size_t no, size_t nd, const size_t* meta, const T* go, T* gi) {
    if (g_wide) pad_backward_impl<T, MODE, typename WideAcc<T>::type>(ni, no, nd, meta, go, gi);
    else pad_backward_impl<T, MODE, T>(ni, no, nd, meta, go, gi);
}
#define DEF_PAD(SUF, T)                                                                                                                        \
    extern "C" void pad_with_constant_##SUF(size_t ni, size_t no, size_t nd, const size_t* m, const T* i, T* o, CArg<T>::type c) {              \
        pad_forward<T, P_CONSTANT>(ni, no, nd, m, i, o, CArg<T>::get(c));                                                                      \
    }                                                                                                                                          \
    extern "C" void pad_with_reflection_##SUF(size_t ni, size_t no, size_t nd, const size_t* m, const T* i, T* o) {                             \
        pad_forward<T, P_REFLECTION>(ni, no, nd, m, i, o, zero_of<T>());                                                                       \
    }                                                                                                                                          \
    extern "C" void pad_with_replication_##SUF(size_t ni, size_t no, size_t nd, const size_t* m, const T* i, T* o) {                            \
        pad_forward<T, P_REPLICATION>(ni, no, nd, m, i, o, zero_of<T>());                                                                      \
    }                                                                                                                                          \
    extern "C" void pad_with_constant_backward_##SUF(size_t ni, size_t no, size_t nd, const size_t* m, const T* g, T* gi) {                     \
        pad_backward<T, P_CONSTANT>(ni, no, nd, m, g, gi);                                                                                     \
    }                                                                                                                                          \
    extern "C" void pad_with_reflection_backward_##SUF(size_t ni, size_t no, size_t nd, const size_t* m, const T* g, T* gi) {                   \
        pad_backward<T, P_REFLECTION>(ni, no, nd, m, g, gi);                                                                                   \
    }                                                                                                                                          \
    extern "C" void pad_with_replication_backward_##SUF(size_t ni, size_t no, size_t nd, const size_t* m, const T* g, T* gi) {                  \
        pad_backward<T, P_REPLICATION>(ni, no, nd, m, g, gi);                                                                                  \
    }
FOR_ARITH12(DEF_PAD)

// ---------------------------------------------------------------------------------
// softmax: crates/maidenx_cpu/src/nn/activation/softmax.rs:63-217
// metadata: [dims(n) | strides(n) | offset]; every step (x - max, exp, the running sum, the quotient) is
// carried out in the element type, as the reference's generic code does for bf16 / f16.
// ---------------------------------------------------------------------------------
template <class T>
static inline T sm_exp(T v) {
    if constexpr (is_half_v<T>) return T::from_f32(std::exp(v.to_f32()));
    else return std::exp(v);
}
template <class T>
static inline T sm_neg_inf() {
    if constexpr (is_half_v<T>) return T::from_f32(-INFINITY);
    else return (T)-INFINITY;
}
// wide mode: f32 (f64 for f32 inputs) arithmetic with one final rounding
template <class T, class A>
static void softmax_impl(size_t num_els, size_t nd, size_t dim_in, const size_t* meta, const T* input, T* output) {
    (void)num_els;
    if (!meta || !input || !output || nd == 0) return;
    const size_t dim = dim_in >= nd ? nd - 1 : dim_in;  // :70
    const size_t* dims = meta;
    const size_t* strides = meta + nd;
    const size_t offset = meta[2 * nd];
    size_t pre = 1, post = 1;
    for (size_t d = 0; d < dim; d++) pre *= dims[d];
    for (size_t d = dim + 1; d < nd; d++) post *= dims[d];
    const size_t n = dims[dim];
    bool cont = true;  // :86-98: unlike utils.rs this test does not skip size-1 dims
    {
        size_t acc = 1;
        for (size_t d = nd; d-- > 0;) {
            if (strides[d] != acc) {
                cont = false;
                break;
            }
            acc *= dims[d];
        }
    }
    auto index = [&](size_t pre_idx, size_t i, size_t post_idx) -> size_t {
        if (cont) return offset + pre_idx * (n * post) + i * post + post_idx;
        size_t idx = offset, rem = pre_idx;
        for (size_t d = 0; d < dim; d++) {  // :123-128: ascending dims take the remainders (dim 0 varies fastest)
            idx += (rem % dims[d]) * strides[d];
            rem /= dims[d];
        }
        idx += i * strides[dim];
        rem = post_idx;
        for (size_t d = nd; d-- > dim + 1;) {
            idx += (rem % dims[d]) * strides[d];
            rem /= dims[d];
        }
        return idx;
    };
#pragma omp parallel for schedule(static)
    for (long long s = 0; s < (long long)(pre * post); s++) {
        const size_t pre_idx = (size_t)s / post, post_idx = (size_t)s % post;
        if constexpr (std::is_same<A, T>::value) {
            T mx = sm_neg_inf<T>();
            for (size_t i = 0; i < n; i++) {
                T v = input[index(pre_idx, i, post_idx)];
                if (v > mx) mx = v;
            }
            T sum = sm_exp<T>(sm_neg_inf<T>() - mx);  // :144
            for (size_t i = 0; i < n; i++) sum = sum + sm_exp<T>(input[index(pre_idx, i, post_idx)] - mx);
            for (size_t i = 0; i < n; i++) output[pre_idx * (n * post) + i * post + post_idx] = sm_exp<T>(input[index(pre_idx, i, post_idx)] - mx) / sum;
        } else {
            A mx = (A)-INFINITY;
            for (size_t i = 0; i < n; i++) {
                A v = to_acc<A, T>(input[index(pre_idx, i, post_idx)]);
                if (v > mx) mx = v;
            }
            A sum = std::exp((A)-INFINITY - mx);
            for (size_t i = 0; i < n; i++) sum += std::exp(to_acc<A, T>(input[index(pre_idx, i, post_idx)]) - mx);
            for (size_t i = 0; i < n; i++)
                output[pre_idx * (n * post) + i * post + post_idx] = from_acc<T, A>(std::exp(to_acc<A, T>(input[index(pre_idx, i, post_idx)]) - mx) / sum);
        }
    }
}
template <class T>
static void softmax_op(size_t n, size_t nd, size_t dim, const size_t* meta, const T* in, T* out) {
    if (g_wide) softmax_impl<T, typename WideAcc<T>::type>(n, nd, dim, meta, in, out);
    else softmax_impl<T, T>(n, nd, dim, meta, in, out);
}
#define DEF_SOFTMAX(SUF, T) \
    extern "C" void softmax_##SUF(size_t n, size_t nd, size_t dim, const size_t* m, const T* i, T* o) { softmax_op<T>(n, nd, dim, m, i, o); }
FOR_FLOAT4(DEF_SOFTMAX)

// ---------------------------------------------------------------------------------
// dtype casts: crates/maidenx_core/src/buffer/mod.rs:132-575 (copy_from_with_dtype_cast).  Element rules:
//   16-bit float -> X        to_f32(x) `as` X (float -> int saturates, NaN -> 0); -> bool: to_f32(x) != 0   (:330-378)
//   f32 / f64 -> 16-bit      from_f32(x as f32): an f64 is rounded to f32 first                              (:281-302)
//   f32 / f64 -> int, float  Rust `as`                                                                       (:152-196)
//   anything -> bool         x != 0 (a NaN is true)                                                          (:260-280)
//   bool -> X                through u8 (0 / 1)
//   u8 / i8 -> 16-bit float  exact (`From`);  wider integers -> 16-bit float go through `as u8` / `as i8` FIRST, i.e. only
//                            their low byte survives (:93-94, :107-108, :121-122, :149-150, :163-164, :177-178)
//   int -> int               Rust `as`: truncate or sign-/zero-extend
// ---------------------------------------------------------------------------------
template <class From, class To>
static inline To cast_one(From x) {
    if constexpr (std::is_same<From, To>::value) {
        return x;
    } else if constexpr (std::is_same<To, bool>::value) {
        if constexpr (is_half_v<From>) return x.to_f32() != 0.0f;
        else return x != (From)0;
    } else if constexpr (is_half_v<From>) {
        const f32 v = x.to_f32();
        if constexpr (is_half_v<To>) return To::from_f32(v);
        else if constexpr (std::is_floating_point<To>::value) return (To)v;
        else return sat_cast<To, f32>(v);
    } else if constexpr (is_half_v<To>) {
        if constexpr (std::is_floating_point<From>::value) return To::from_f32((f32)x);
        else if constexpr (std::is_same<From, bool>::value) return To::from_f32(x ? 1.0f : 0.0f);
        else if constexpr (std::is_signed<From>::value) return To::from_f32((f32)(int8_t)x);   // `as i8`, then From<i8>
        else return To::from_f32((f32)(uint8_t)x);                                             // `as u8`, then From<u8>
    } else if constexpr (std::is_floating_point<From>::value) {
        if constexpr (std::is_floating_point<To>::value) return (To)x;
        else return sat_cast<To, From>(x);
    } else if constexpr (std::is_same<From, bool>::value) {
        return (To)(uint8_t)(x ? 1 : 0);
    } else {
        return (To)x;  // integer source: value-preserving to floats (round to nearest), modular to integers
    }
}
template <class From, class To>
static void cast_op(size_t n, const From* in, To* out) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++) out[i] = cast_one<From, To>(in[i]);
}
#define DEF_CAST_TO(TSUF, TO, FSUF, FROM) \
    extern "C" void cast_##FSUF##_##TSUF(size_t n, const FROM* i, TO* o) { cast_op<FROM, TO>(n, i, o); }
// (a second copy of the dtype list: a macro cannot expand inside its own expansion)
#define CAST_TARGETS(X, ...)                                                                                                                 \
    X(bf16, bf16, ##__VA_ARGS__) X(f16, f16, ##__VA_ARGS__) X(f32, f32, ##__VA_ARGS__) X(f64, f64, ##__VA_ARGS__) X(bool, bool, ##__VA_ARGS__) \
    X(u8, u8, ##__VA_ARGS__) X(u16, u16, ##__VA_ARGS__) X(u32, u32, ##__VA_ARGS__) X(u64, u64, ##__VA_ARGS__)                                \
    X(i8, i8, ##__VA_ARGS__) X(i16, i16, ##__VA_ARGS__) X(i32, i32, ##__VA_ARGS__) X(i64, i64, ##__VA_ARGS__)
#define DEF_CAST_FROM(FSUF, FROM) CAST_TARGETS(DEF_CAST_TO, FSUF, FROM)
FOR_ALL13(DEF_CAST_FROM)
