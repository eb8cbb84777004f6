// C-ABI entry points of the reduction family for one dtype (MX_T).
// Replaces the symbols declared in crates/maidenx_cuda/src/ops/reduction.rs:6-104 that the
// reference's dispatch uses: sum, max, min, sum_to_shape (12 dtypes) and mean (floats).
#include "abi_common.cuh"
#include "reduction.cuh"

#ifndef MX_T
#error "compile with -DMX_T=<dtype suffix> -DMX_TCLASS=<class>"
#endif

#define DEF_REDUCE_(op, KIND, T)                                                                                    \
    void cuda_##op##_##T(size_t n, size_t nd, size_t nr, const size_t* m, const mx_##T* i, mx_##T* o) {             \
        mx::reduce_entry<mx_##T, mx::KIND>(n, nd, nr, m, i, o, "cuda_" #op "_" #T);                                 \
    }
#define DEF_REDUCE(op, KIND, T) DEF_REDUCE_(op, KIND, T)
#define DEF_STS_(T)                                                                                                 \
    void cuda_sum_to_shape_##T(size_t n, size_t nd, const size_t* m, const mx_##T* i, mx_##T* o) {                  \
        mx::sum_to_shape_entry<mx_##T>(n, nd, m, i, o, "cuda_sum_to_shape_" #T);                                    \
    }
#define DEF_STS(T) DEF_STS_(T)

extern "C" {
DEF_REDUCE(sum, RED_SUM, MX_T)
DEF_REDUCE(max, RED_MAX, MX_T)
DEF_REDUCE(min, RED_MIN, MX_T)
DEF_STS(MX_T)
#if MX_TCLASS == MX_CLASS_FLOAT
DEF_REDUCE(mean, RED_MEAN, MX_T)
#endif
}
