// Host-side parsing of the matmul metadata block and construction of the index functions
// the SIMT kernel evaluates (see matmul_simt.cuh).
#include "matmul_simt.cuh"

namespace mx {

size_t mm_meta_words(const size_t* h) { return 3 + h[0] + 2 * h[1] + 2 * h[2] + 2; }

namespace {
bool contiguous(size_t nd, const size_t* dims, const size_t* strides) {
    size_t acc = 1;
    for (size_t d = nd; d-- > 0;) {
        if (dims[d] > 1 && strides[d] != acc) return false;
        acc *= dims[d];
    }
    return true;
}
}  // namespace

bool mm_parse(const size_t* hm, MmDesc& d) {
    d.valid = false;
    d.out_nd = hm[0];
    d.a_nd = hm[1];
    d.b_nd = hm[2];
    if (d.a_nd == 0 || d.b_nd == 0) return false;  // crates/maidenx_cpu/src/ops/matmul.rs:28-30
    const size_t* out_shape = hm + 3;
    const size_t* a_shape = out_shape + d.out_nd;
    const size_t* b_shape = a_shape + d.a_nd;
    const size_t* a_st = b_shape + d.b_nd;
    const size_t* b_st = a_st + d.a_nd;
    d.a_off = b_st[d.b_nd];
    d.b_off = b_st[d.b_nd + 1];
    d.m = d.out_nd >= 2 ? out_shape[d.out_nd - 2] : 1;
    d.n = d.out_nd >= 1 ? out_shape[d.out_nd - 1] : 1;
    d.k_fwd = a_shape[d.a_nd - 1];
    d.k_bwd = d.b_nd >= 2 ? b_shape[d.b_nd - 2] : a_shape[d.a_nd - 1];  // matmul.rs:170-176
    d.g_size = 1;
    for (size_t i = 0; i < d.out_nd; i++) d.g_size *= out_shape[i];
    d.a_cont = contiguous(d.a_nd, a_shape, a_st);
    d.b_cont = contiguous(d.b_nd, b_shape, b_st);
    if (d.a_nd >= 2) {
        d.a_strides[0] = (int64_t)a_st[0];
        d.a_strides[1] = (int64_t)a_st[d.a_nd - 2];
        d.a_strides[2] = (int64_t)a_st[d.a_nd - 1];
    } else {
        d.a_strides[0] = d.a_strides[1] = 0;
        d.a_strides[2] = (int64_t)a_st[0];
    }
    if (d.b_nd >= 2) {
        d.b_strides[0] = (int64_t)b_st[0];
        d.b_strides[1] = (int64_t)b_st[d.b_nd - 2];
        d.b_strides[2] = (int64_t)b_st[d.b_nd - 1];
    } else {  // rank-1 B is indexed by the output column only (matmul.rs:101-103)
        d.b_strides[0] = d.b_strides[1] = 0;
        d.b_strides[2] = (int64_t)b_st[0];
    }
    d.valid = true;
    return true;
}

}  // namespace mx
