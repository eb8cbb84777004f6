// C-ABI entry points of the binary elementwise family for one dtype (MX_T).
// Replaces the symbols declared in crates/maidenx_cuda/src/ops/binary.rs:6-182.
#include "abi_common.cuh"
#include "elementwise.cuh"
#include "ops.cuh"

#ifndef MX_T
#error "compile with -DMX_T=<dtype suffix> -DMX_TCLASS=<class>"
#endif

namespace mx {
typedef OpAdd Op_add;
typedef OpSub Op_sub;
typedef OpMul Op_mul;
typedef OpDiv Op_div;
typedef OpMax Op_maximum;
typedef OpMin Op_minimum;
typedef OpLAnd Op_logical_and;
typedef OpLOr Op_logical_or;
typedef OpLXor Op_logical_xor;
typedef OpEq Op_eq;
typedef OpNe Op_ne;
typedef OpLt Op_lt;
typedef OpLe Op_le;
typedef OpGt Op_gt;
typedef OpGe Op_ge;
typedef OpAdd Op_add_inplace;
typedef OpSub Op_sub_inplace;
typedef OpMul Op_mul_inplace;
typedef OpDiv Op_div_inplace;
}  // namespace mx

#define DEF_BINARY_(op, T)                                                                                                             \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, const mx_##T* l, const mx_##T* r, mx_##T* o) {                          \
        mx::binary_entry<mx::Op_##op, mx_##T, mx_##T>(n, nd, m, l, r, o, false, "cuda_" #op "_" #T);                                   \
    }
#define DEF_BINARY_BOOL_(op, T)                                                                                                        \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, const mx_##T* l, const mx_##T* r, mx_bool* o) {                         \
        mx::binary_entry<mx::Op_##op, mx_##T, bool>(n, nd, m, l, r, o, false, "cuda_" #op "_" #T);                                     \
    }
#define DEF_BINARY_INPLACE_(op, T)                                                                                                     \
    void cuda_##op##_##T(size_t n, size_t nd, const size_t* m, mx_##T* l, const mx_##T* r) {                                           \
        mx::binary_entry<mx::Op_##op, mx_##T, mx_##T>(n, nd, m, l, r, l, true, "cuda_" #op "_" #T);                                    \
    }
#define DEF_BINARY(op, T) DEF_BINARY_(op, T)
#define DEF_BINARY_BOOL(op, T) DEF_BINARY_BOOL_(op, T)
#define DEF_BINARY_INPLACE(op, T) DEF_BINARY_INPLACE_(op, T)

extern "C" {
#if MX_TCLASS != MX_CLASS_BOOL
MX_BINARY_ARITH_OPS(DEF_BINARY, MX_T)
MX_BINARY_INPLACE_OPS(DEF_BINARY_INPLACE, MX_T)
#endif
MX_BINARY_BOOL_OPS(DEF_BINARY_BOOL, MX_T)
}
