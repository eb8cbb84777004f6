// C-ABI entry points of the unary and unary-with-constant families for one dtype (MX_T).
// Replaces the symbols declared in crates/maidenx_cuda/src/ops/unary.rs:6-192; the dtype
// coverage per op is the one maidenx_core dispatches
// (crates/maidenx_core/src/be/ops/unary.rs:486-526).
#include "abi_common.cuh"
#include "elementwise.cuh"
#include "ops.cuh"

#ifndef MX_T
#error "compile with -DMX_T=<dtype suffix> -DMX_TCLASS=<class>"
#endif

namespace mx {
typedef OpRelu Op_relu;
typedef OpSigmoid Op_sigmoid;
typedef OpTanh Op_tanh;
typedef OpGelu Op_gelu;
typedef OpSin Op_sin;
typedef OpCos Op_cos;
typedef OpTan Op_tan;
typedef OpLn Op_ln;
typedef OpLog10 Op_log10;
typedef OpLog2 Op_log2;
typedef OpExp Op_exp;
typedef OpExp10 Op_exp10;
typedef OpExp2 Op_exp2;
typedef OpSoftplus Op_softplus;
typedef OpRecip Op_recip;
typedef OpNeg Op_neg;
typedef OpAbs Op_abs;
typedef OpSign Op_sign;
typedef OpSquare Op_square;
typedef OpSqrt Op_sqrt;
typedef OpLogicalNot Op_logical_not;
typedef OpAdd Op_add_scalar;
typedef OpSub Op_sub_scalar;
typedef OpMul Op_mul_scalar;
typedef OpDiv Op_div_scalar;
typedef OpMax Op_maximum_scalar;
typedef OpMin Op_minimum_scalar;
typedef OpPow Op_pow;
typedef OpLeakyRelu Op_leaky_relu;
typedef OpElu Op_elu;
typedef OpEq Op_eq_scalar;
typedef OpNe Op_ne_scalar;
typedef OpLt Op_lt_scalar;
typedef OpLe Op_le_scalar;
typedef OpGt Op_gt_scalar;
typedef OpGe Op_ge_scalar;
typedef OpIdentity Op_contiguous;
}  // namespace mx

#define DEF_UNARY_(op, T)                                                                                          \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o) {                       \
        mx::unary_entry<mx::Op_##op, mx_##T, mx_##T>(n, nd, m, i, o, "cuda_" #op "_" #T);                          \
    }
#define DEF_UNARY_BOOL_(op, T)                                                                                     \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_bool* o) {                      \
        mx::unary_entry<mx::Op_##op, mx_##T, bool>(n, nd, m, i, o, "cuda_" #op "_" #T);                            \
    }
#define DEF_UNARY_CONST_(op, T)                                                                                    \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_##T##_arg c, mx_##T* o) {       \
        mx::unary_const_entry<mx::Op_##op, mx_##T, mx_##T>(n, nd, m, i, mx::scalar_arg<mx_##T>(c), o, "cuda_" #op "_" #T); \
    }
#define DEF_UNARY_CONST_BOOL_(op, T)                                                                               \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_##T##_arg c, mx_bool* o) {      \
        mx::unary_const_entry<mx::Op_##op, mx_##T, bool>(n, nd, m, i, mx::scalar_arg<mx_##T>(c), o, "cuda_" #op "_" #T); \
    }
// additive: Tensor::contiguous() on the device (the reference round-trips through the host, crates/maidenx_tensor/src/f.rs:11-40)
#define DEF_CONTIGUOUS_(T)                                                                                         \
    void mx_contiguous_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o) {                     \
        mx::unary_entry<mx::Op_contiguous, mx_##T, mx_##T>(n, nd, m, i, o, "mx_contiguous_" #T);                   \
    }
#define DEF_CONTIGUOUS(T) DEF_CONTIGUOUS_(T)
#define DEF_UNARY(op, T) DEF_UNARY_(op, T)
#define DEF_UNARY_BOOL(op, T) DEF_UNARY_BOOL_(op, T)
#define DEF_UNARY_CONST(op, T) DEF_UNARY_CONST_(op, T)
#define DEF_UNARY_CONST_BOOL(op, T) DEF_UNARY_CONST_BOOL_(op, T)

extern "C" {
#if MX_TCLASS == MX_CLASS_FLOAT
MX_UNARY_FLOAT_OPS(DEF_UNARY, MX_T)
MX_UNARY_CONST_FLOAT_OPS(DEF_UNARY_CONST, MX_T)
#endif
#if MX_TCLASS == MX_CLASS_FLOAT || MX_TCLASS == MX_CLASS_SINT
MX_UNARY_SIGNED_OPS(DEF_UNARY, MX_T)
#endif
#if MX_TCLASS != MX_CLASS_BOOL
MX_UNARY_ARITH_OPS(DEF_UNARY, MX_T)
MX_UNARY_CONST_ARITH_OPS(DEF_UNARY_CONST, MX_T)
#endif
DEF_UNARY_BOOL(logical_not, MX_T)
MX_UNARY_CONST_BOOL_OPS(DEF_UNARY_CONST_BOOL, MX_T)
DEF_CONTIGUOUS(MX_T)
}
