// C-ABI entry points of matmul / matmul_backward for one dtype (MX_T).
// Replaces the symbols declared in crates/maidenx_cuda/src/ops/matmul.rs:6-50.
#include "abi_common.cuh"
#include "matmul_simt.cuh"
#include "matmul_tc.cuh"

#ifndef MX_T
#error "compile with -DMX_T=<dtype suffix> -DMX_TCLASS=<class>"
#endif

namespace mx {

template <class T>
void matmul_entry(size_t num_els, const size_t* meta, const T* a, const T* b, T* c, const char* where) {
    if (!meta || !a || !b || !c) return;  // crates/maidenx_cpu/src/ops/matmul.rs:20-22
    const size_t* h3 = resolve_metadata(meta, 3);
    if (!h3) return;
    size_t words = mm_meta_words(h3);
    const size_t* hm = resolve_metadata(meta, words);
    if (!hm) return;
    MmDesc d;
    if (!mm_parse(hm, d)) return;
    if (d.m == 0 || d.n == 0 || d.k_fwd == 0 || num_els == 0) return;
    if (tc_matmul_forward<T>(d, num_els, a, b, c, where)) return;
    MmParams P;
    P.rows = (num_els + d.n - 1) / d.n;
    P.N = d.n;
    P.K = d.k_fwd;
    P.M = d.m;
    P.out_elems = num_els;
    if (d.a_cont && d.b_cont) {
        P.xs_b = (int64_t)(d.m * d.k_fwd);
        P.xs_m = (int64_t)d.k_fwd;
        P.xs_r = 1;
        P.ys_b = (int64_t)(d.k_fwd * d.n);
        P.ys_r = (int64_t)d.n;
        P.ys_c = 1;
    } else {
        P.xs_b = d.a_strides[0];
        P.xs_m = d.a_strides[1];
        P.xs_r = d.a_strides[2];
        P.ys_b = d.b_strides[0];
        P.ys_r = d.b_strides[1];
        P.ys_c = d.b_strides[2];
    }
    P.x_limit = P.y_limit = (uint64_t)num_els * d.k_fwd;  // matmul.rs:55-56
    mm_launch<T>(P, a + d.a_off, b + d.b_off, c, where);
}

template <class T>
void matmul_backward_entry(size_t nea, size_t neb, const size_t* meta, const T* g, const T* a, const T* b, T* ga, T* gb, const char* where) {
    if (!meta || !g || !a || !b) return;  // matmul.rs:146-148
    const size_t* h3 = resolve_metadata(meta, 3);
    if (!h3) return;
    const size_t* hm = resolve_metadata(meta, mm_meta_words(h3));
    if (!hm) return;
    MmDesc d;
    if (!mm_parse(hm, d)) return;
    const uint64_t m = d.m, n = d.n, k = d.k_bwd;
    if (m == 0 || n == 0 || k == 0 || d.g_size == 0) return;
    const bool scalar_g = d.out_nd == 0;
    if (ga && nea) {
        if (!tc_matmul_grad_a<T>(d, nea, neb, g, b + d.b_off, ga, where)) {
            MmParams P;
            P.rows = (nea + k - 1) / k;
            P.N = k;
            P.M = m;
            P.out_elems = nea;
            if (scalar_g) {  // matmul.rs:204-207
                P.K = 1;
                P.xs_b = P.xs_m = P.xs_r = 0;
                P.x_limit = 1;
                P.ys_b = P.ys_r = 0;
                P.ys_c = 1;
            } else {         // matmul.rs:208-216
                P.K = n;
                P.xs_b = (int64_t)(m * n);
                P.xs_m = (int64_t)n;
                P.xs_r = 1;
                P.x_limit = d.g_size;
                P.ys_b = (int64_t)(k * n);
                P.ys_r = 1;
                P.ys_c = (int64_t)n;
            }
            P.y_limit = neb;
            mm_launch<T>(P, g, b + d.b_off, ga, where);
        }
    }
    if (gb && neb) {
        if (!tc_matmul_grad_b<T>(d, nea, neb, g, a + d.a_off, gb, where)) {
            MmParams P;
            P.rows = (neb + n - 1) / n;
            P.N = n;
            P.M = k;
            P.out_elems = neb;
            if (scalar_g) {  // matmul.rs:240-243
                P.K = 1;
                P.xs_b = P.xs_r = 0;
                P.xs_m = 1;
                P.ys_b = P.ys_r = P.ys_c = 0;
                P.y_limit = 1;
            } else {         // matmul.rs:244-256
                P.K = m;
                P.xs_b = (int64_t)(m * k);
                P.xs_m = 1;
                P.xs_r = (int64_t)k;
                P.ys_b = (int64_t)(m * n);
                P.ys_r = (int64_t)n;
                P.ys_c = 1;
                P.y_limit = d.g_size;
            }
            P.x_limit = nea;
            mm_launch<T>(P, a + d.a_off, g, gb, where);
        }
    }
}

}  // namespace mx

#define DEF_MM_(T)                                                                                                           \
    void cuda_matmul_##T(size_t n, const size_t* m, const mx_##T* a, const mx_##T* b, mx_##T* c) {                           \
        mx::matmul_entry<mx_##T>(n, m, a, b, c, "cuda_matmul_" #T);                                                          \
    }                                                                                                                        \
    void cuda_matmul_backward_##T(size_t na, size_t nb, const size_t* m, const mx_##T* g, const mx_##T* a, const mx_##T* b,  \
                                  mx_##T* ga, mx_##T* gb) {                                                                  \
        mx::matmul_backward_entry<mx_##T>(na, nb, m, g, a, b, ga, gb, "cuda_matmul_backward_" #T);                           \
    }
#define DEF_MM(T) DEF_MM_(T)

extern "C" {
DEF_MM(MX_T)
}
