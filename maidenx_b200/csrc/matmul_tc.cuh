// Interface between the matmul entry points and the tensor-core (tcgen05) path.
// Each function returns true when it handled the product; false sends the call to the
// SIMT kernel.  Only bf16 / f16 have a tensor-core implementation.
#pragma once
#include "matmul_simt.cuh"

namespace mx {

bool tc_gemm_bf16_f16(bool is_bf16, const MmDesc& d, int which, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, void* out,
                      const char* where);

template <class T>
inline bool tc_matmul_forward(const MmDesc& d, size_t num_els, const T* a, const T* b, T* c, const char* where) {
    if constexpr (is_half_v<T>) return tc_gemm_bf16_f16(std::is_same<T, bf16>::value, d, 0, num_els, 0, 0, a, b, c, where);
    else return false;
}
template <class T>
inline bool tc_matmul_grad_a(const MmDesc& d, size_t nea, size_t neb, const T* g, const T* b_off, T* ga, const char* where) {
    if constexpr (is_half_v<T>) return tc_gemm_bf16_f16(std::is_same<T, bf16>::value, d, 1, 0, nea, neb, g, b_off, ga, where);
    else return false;
}
template <class T>
inline bool tc_matmul_grad_b(const MmDesc& d, size_t nea, size_t neb, const T* g, const T* a_off, T* gb, const char* where) {
    if constexpr (is_half_v<T>) return tc_gemm_bf16_f16(std::is_same<T, bf16>::value, d, 2, 0, nea, neb, g, a_off, gb, where);
    else return false;
}

}  // namespace mx
