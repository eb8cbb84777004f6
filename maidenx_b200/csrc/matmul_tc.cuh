// Interface between the matmul entry points and the tensor-core (tcgen05) kernels.
// Each function returns true when it handled the product; false sends the call to the
// SIMT kernel.  bf16 / f16 run on kind::f16 (matmul_tc.cu), f32 on split-operand kind::tf32
// (matmul_tc_f32.cu); every other dtype has no tensor-core implementation.
#pragma once
#include "matmul_simt.cuh"

namespace mx {

// A product the tensor-core kernels accept: D[m, n] = sum_k Aop[m, k] * Bop[n, k] with dense operands that are
// K-major ([MN, K] row-major) or MN-major ([K, MN] row-major).
struct TcProduct {
    const char* A;
    const char* B;
    bool a_mn, b_mn;
    uint64_t m, n, k;
    uint64_t batch;      // independent products; D is dense [batch, m, n]
    int64_t a_bs, b_bs;  // elements between consecutive batches of each operand; 0 = one matrix shared by all
};
// which: 0 forward, 1 grad_a, 2 grad_b (see matmul_tc.cu); elem_size in bytes.
bool tc_classify(const MmDesc& d, int which, size_t elem_size, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, const void* out,
                 TcProduct& c);

bool tc_gemm_bf16_f16(bool is_bf16, const MmDesc& d, int which, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, void* out,
                      const char* where);
// Linear forward with its bias add and activation folded into the product's epilogue (bf16 / f16): u = x . w^T + bias and,
// when `act` is not NULL, act = gelu(u), each rounded exactly as the separate ops round.  `bias` is one element in device
// memory.  Returns false when the shape does not qualify for the tensor-core kernel; nothing was launched then.
bool tc_linear_bias_act(bool is_bf16, uint64_t rows, uint64_t in_features, uint64_t out_features, const void* x, const void* w, const void* bias,
                        void* u, void* act, const char* where);
// Batched product with a per-row bias in the epilogue (bf16 / f16): out[b] = w[rows, k] . cols[b][k, n] + bias[rows], the
// form of a convolution's forward pass over its column buffer.  false = not taken by the tensor-core kernel, nothing launched.
bool tc_batched_row_bias(bool is_bf16, uint64_t batch, uint64_t rows, uint64_t k, uint64_t n, const void* w, const void* cols, const void* bias, void* out,
                         const char* where);
bool tc_gemm_f32(const MmDesc& d, int which, size_t num_els, size_t nea, size_t neb, const void* x, const void* y, void* out, const char* where);

template <class T>
inline bool tc_dispatch(const MmDesc& d, int which, size_t num_els, size_t nea, size_t neb, const T* x, const T* y, T* out, const char* where) {
    if constexpr (is_half_v<T>) return tc_gemm_bf16_f16(std::is_same<T, bf16>::value, d, which, num_els, nea, neb, x, y, out, where);
    else if constexpr (std::is_same<T, float>::value) return tc_gemm_f32(d, which, num_els, nea, neb, x, y, out, where);
    else return false;
}
template <class T>
inline bool tc_matmul_forward(const MmDesc& d, size_t num_els, const T* a, const T* b, T* c, const char* where) {
    return tc_dispatch<T>(d, 0, num_els, 0, 0, a, b, c, where);
}
template <class T>
inline bool tc_matmul_grad_a(const MmDesc& d, size_t nea, size_t neb, const T* g, const T* b_off, T* ga, const char* where) {
    return tc_dispatch<T>(d, 1, 0, nea, neb, g, b_off, ga, where);
}
template <class T>
inline bool tc_matmul_grad_b(const MmDesc& d, size_t nea, size_t neb, const T* g, const T* a_off, T* gb, const char* where) {
    return tc_dispatch<T>(d, 2, 0, nea, neb, g, a_off, gb, where);
}

}  // namespace mx
