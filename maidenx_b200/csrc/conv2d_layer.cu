// Conv2d forward and backward composed from the op layer's own entry points, the way the reference's layer
// composes them (crates/maidenx_nn/src/layers/conv.rs:185-307 with the im2col / col2im wrappers at :333-420):
// im2col -> matmul -> (views) -> bias add, and in backward matmul -> col2im for the input gradient, matmul for
// the weight gradient and three sums for the bias gradient.  Every step is a call of a cuda_<op>_<dtype> symbol of
// this library with the metadata the reference's tensor layer would build; nothing here launches a kernel itself.
//
// Two compositions are offered (argument `mode`):
//
//   0  "as the reference calls it".  The layer hands the ops a column buffer it declares as [B*oh*ow, C*kh*kw]
//      although im2col writes it as [B][C*kh*kw][oh*ow]; it passes (stride, padding) in the metadata slots where
//      the kernels read (padding, stride); col2im gets num_els = B*C*H*W, so it reads only that many column
//      entries; and the [C*kh*kw, Cout] weight gradient is re-labelled [Cout, C, kh, kw] without a transpose.
//      This mode reproduces those calls literally: it is what an unchanged maidenx_nn would execute on this
//      library, and it is the parity target for the call sequence.  (With stride == padding the slot swap is
//      invisible; the buffer re-labelling is not, so its results are not a convolution.)
//   1  "direct".  The same ops used consistently: the column buffer is read as the [B][K][P] array im2col
//      wrote, so out[b] = W[Cout, K] . cols[b][K, P] is one batched product with the weight shared by every
//      batch (a stride-0 leading dim, which is how Tensor::matmul broadcasts, crates/maidenx_tensor/src/ops/
//      matmul.rs:161-225); grad_cols[b] = W^T . g[b]; col2im reads the whole buffer; grad_W = sum_b g[b] . cols[b]^T.
//      This mode is a convolution and is checked against a direct f64 convolution.
//
// The caller owns every buffer, as everywhere in this ABI: `cols` (B*P*K elements) is written by forward and read
// by backward; `workspace` holds the intermediates (sizes from mx_conv2d_workspace_elems).
#include "abi_common.cuh"
#include "matmul_tc.cuh"

namespace mx {

template <class T>
constexpr int half_kind_of() {
    return std::is_same<T, bf16>::value ? 1 : (std::is_same<T, f16>::value ? 2 : 0);
}

namespace {

struct Geometry {
    size_t B, C, H, W, Co, kh, kw, sh, sw, ph, pw, oh, ow, P, K;
};

bool geometry(const MxConv2d* c, Geometry& g) {
    if (!c || !c->batch || !c->in_channels || !c->out_channels || !c->kernel_h || !c->kernel_w || !c->stride_h || !c->stride_w) return false;
    g.B = c->batch;
    g.C = c->in_channels;
    g.H = c->height;
    g.W = c->width;
    g.Co = c->out_channels;
    g.kh = c->kernel_h;
    g.kw = c->kernel_w;
    g.sh = c->stride_h;
    g.sw = c->stride_w;
    g.ph = c->pad_h;
    g.pw = c->pad_w;
    if (g.H + 2 * g.ph < g.kh || g.W + 2 * g.pw < g.kw) return false;
    g.oh = (g.H + 2 * g.ph - g.kh) / g.sh + 1;  // conv.rs:198-199
    g.ow = (g.W + 2 * g.pw - g.kw) / g.sw + 1;
    g.P = g.oh * g.ow;
    g.K = g.C * g.kh * g.kw;
    return true;
}

size_t round16(size_t elems) { return (elems + 15) & ~(size_t)15; }  // keeps every sub-buffer 16-byte aligned for any dtype

// The op entry points of one dtype, with untyped pointers.
struct Ops {
    void (*im2col)(size_t, const size_t*, const void*, void*);
    void (*col2im)(size_t, const size_t*, const void*, void*);
    void (*matmul)(size_t, const size_t*, const void*, const void*, void*);
    void (*add)(size_t, size_t, const size_t*, const void*, const void*, void*);
    void (*add_inplace)(size_t, size_t, const size_t*, void*, const void*);
    void (*sum)(size_t, size_t, size_t, const size_t*, const void*, void*);
    void (*contiguous)(size_t, size_t, const size_t*, const void*, void*);
    int half_kind;  // 1 bf16, 2 f16, 0 anything else
};
#define MX_CONV_OPS(T)                                                                                                                  \
    mx::Ops {                                                                                                                           \
        reinterpret_cast<decltype(mx::Ops::im2col)>(cuda_conv2d_im2col_##T), reinterpret_cast<decltype(mx::Ops::col2im)>(cuda_conv2d_col2im_##T), \
            reinterpret_cast<decltype(mx::Ops::matmul)>(cuda_matmul_##T), reinterpret_cast<decltype(mx::Ops::add)>(cuda_add_##T),                 \
            reinterpret_cast<decltype(mx::Ops::add_inplace)>(cuda_add_inplace_##T), reinterpret_cast<decltype(mx::Ops::sum)>(cuda_sum_##T),        \
            reinterpret_cast<decltype(mx::Ops::contiguous)>(mx_contiguous_##T), mx::half_kind_of<mx_##T>()                                       \
    }

// sum over one dim of a dense tensor, metadata as crates/maidenx_tensor/src/ops/reduction.rs:722-733 builds it
void sum_dim(const Ops& ops, const size_t* dims, size_t nd, size_t dim, const void* in, void* out) {
    size_t meta[2 * 8 + 3], strides[8], n = 1;
    for (size_t d = nd; d-- > 0;) {
        strides[d] = n;
        n *= dims[d];
    }
    for (size_t d = 0; d < nd; d++) {
        meta[d] = dims[d];
        meta[nd + d] = strides[d];
    }
    meta[2 * nd] = dims[dim];
    meta[2 * nd + 1] = strides[dim];
    meta[2 * nd + 2] = 0;
    ops.sum(n, nd, 1, meta, in, out);
}

// grad_bias = grad_out.sum(3).sum(2).sum(0) (conv.rs:283-288); tmp holds B*Co*oh + B*Co elements
void bias_gradient(const Ops& ops, const Geometry& g, size_t es, const void* grad_out, char* tmp, void* grad_bias) {
    const size_t d4[4] = {g.B, g.Co, g.oh, g.ow}, d3[3] = {g.B, g.Co, g.oh}, d2[2] = {g.B, g.Co};
    char* t1 = tmp;
    char* t2 = tmp + round16(g.B * g.Co * g.oh) * es;
    sum_dim(ops, d4, 4, 3, grad_out, t1);
    sum_dim(ops, d3, 3, 2, t1, t2);
    sum_dim(ops, d2, 2, 0, t2, grad_bias);
}

size_t workspace_elems(const Geometry& g, int mode, int backward) {
    const size_t sums = round16(g.B * g.Co * g.oh) + round16(g.B * g.Co);
    if (mode == 0) {
        if (!backward) return round16(g.B * g.P * g.Co);                                 // out_flat
        return round16(g.B * g.P * g.Co) + round16(g.B * g.P * g.K) + sums;              // grad_flat, grad_cols, sums
    }
    if (!backward) return 16;
    return round16(g.B * g.K * g.P) + round16(g.B * g.Co * g.K) + sums;                   // grad_cols, per-batch grad_W, sums
}

void forward(const Ops& ops, size_t es, const MxConv2d* c, int mode, const void* x, const void* w, const void* bias, void* cols, void* workspace,
             void* out) {
    Geometry g;
    if (!geometry(c, g) || !x || !w || !cols || !out || (mode == 0 && !workspace)) {
        set_error(kErrBadMetadata, 0, "mx_conv2d_forward");
        return;
    }
    if (mode == 0 && (g.ph == 0 || g.pw == 0)) {
        // the kernels would read the padding as their stride: a zero stride divides by zero in the reference's CPU backend
        set_error(kErrUnsupported, 0, "mx_conv2d_forward");
        return;
    }
    const size_t ncol = g.B * g.P * g.K;
    if (mode == 0) {
        // conv.rs:345-358: stride in the slots the kernels read as padding, and the other way round
        const size_t cm[12] = {g.B, g.C, g.H, g.W, g.kh, g.kw, g.oh, g.ow, g.sh, g.sw, g.ph, g.pw};
        ops.im2col(ncol, cm, x, cols);
        // cols declared [B*P, K] (conv.rs:334-337) . weight_matrix^T, the transposed view of [Co, K] (conv.rs:214-219)
        const size_t M = g.B * g.P;
        const size_t mm[15] = {2, 2, 2, M, g.Co, M, g.K, g.K, g.Co, g.K, 1, 1, g.K, 0, 0};
        ops.matmul(M * g.Co, mm, cols, w, workspace);
        // reshape [B, oh, ow, Co], transpose(1, 3), transpose(2, 3) (conv.rs:221-222): dims [B, Co, oh, ow] over the flat buffer
        const size_t vs[4] = {g.P * g.Co, 1, g.ow * g.Co, g.Co};
        if (bias) {
            // + bias.reshape([1, Co, 1, 1]) (conv.rs:224-228), broadcast = stride 0
            const size_t am[14] = {g.B, g.Co, g.oh, g.ow, vs[0], vs[1], vs[2], vs[3], 0, 1, 0, 0, 0, 0};
            ops.add(g.B * g.Co * g.P, 4, am, workspace, bias, out);
        } else {
            // the reference returns the strided view itself; here the caller gets its dense copy
            const size_t um[9] = {g.B, g.Co, g.oh, g.ow, vs[0], vs[1], vs[2], vs[3], 0};
            ops.contiguous(g.B * g.Co * g.P, 4, um, workspace, out);
        }
        return;
    }
    const size_t cm[12] = {g.B, g.C, g.H, g.W, g.kh, g.kw, g.oh, g.ow, g.ph, g.pw, g.sh, g.sw};
    ops.im2col(ncol, cm, x, cols);
    // out[B, Co, P] = W[Co, K] (shared by every batch) . cols[B, K, P]
    const size_t mm[20] = {3, 3, 3, g.B, g.Co, g.P, g.B, g.Co, g.K, g.B, g.K, g.P, 0, g.K, 1, g.K * g.P, g.P, 1, 0, 0};
    // 16-bit types: the bias add rides in the product's epilogue (same roundings as the two ops below) when the
    // tensor-core kernel takes the shape
    if (bias && ops.half_kind && tc_batched_row_bias(ops.half_kind == 1, g.B, g.Co, g.K, g.P, w, cols, bias, out, "mx_conv2d_forward")) return;
    ops.matmul(g.B * g.Co * g.P, mm, w, cols, out);
    if (bias) {
        const size_t am[11] = {g.B, g.Co, g.P, g.Co * g.P, g.P, 1, 0, 1, 0, 0, 0};
        ops.add_inplace(g.B * g.Co * g.P, 3, am, out, bias);
    }
}

void backward(const Ops& ops, size_t es, const MxConv2d* c, int mode, const void* grad_out, const void* w, const void* cols, void* workspace,
              void* grad_x, void* grad_w, void* grad_bias) {
    Geometry g;
    if (!geometry(c, g) || !grad_out || !w || !cols || !workspace) {
        set_error(kErrBadMetadata, 0, "mx_conv2d_backward");
        return;
    }
    if (mode == 0 && (g.ph == 0 || g.pw == 0)) {
        set_error(kErrUnsupported, 0, "mx_conv2d_backward");
        return;
    }
    char* ws = static_cast<char*>(workspace);
    if (mode == 0) {
        char* grad_flat = ws;
        char* grad_cols = grad_flat + round16(g.B * g.P * g.Co) * es;
        char* sums = grad_cols + round16(g.B * g.P * g.K) * es;
        // grad_out.transpose(2, 3).transpose(1, 3) = dims [B, oh, ow, Co] over the dense [B, Co, oh, ow] buffer, then
        // reshape([B*P, Co]), which copies because the view is not contiguous (conv.rs:250-252)
        const size_t um[9] = {g.B, g.oh, g.ow, g.Co, g.Co * g.P, g.ow, 1, g.P, 0};
        ops.contiguous(g.B * g.P * g.Co, 4, um, grad_out, grad_flat);
        const size_t M = g.B * g.P;
        if (grad_x) {
            // grad_cols[B*P, K] = grad_flat[B*P, Co] . weight_matrix[Co, K] (conv.rs:254)
            const size_t mm[15] = {2, 2, 2, M, g.K, M, g.Co, g.Co, g.K, g.Co, 1, g.K, 1, 0, 0};
            ops.matmul(M * g.K, mm, grad_flat, w, grad_cols);
            // col2im with num_els = B*C*H*W and the same slot order as im2col (conv.rs:390-409)
            const size_t cm[12] = {g.B, g.C, g.H, g.W, g.kh, g.kw, g.oh, g.ow, g.sh, g.sw, g.ph, g.pw};
            ops.col2im(g.B * g.C * g.H * g.W, cm, grad_cols, grad_x);
        }
        if (grad_w) {
            // cols.transpose(-1, -2)[K, B*P] . grad_flat[B*P, Co] (conv.rs:277); the [K, Co] result is what the layer
            // then labels [Co, C, kh, kw]
            const size_t mm[15] = {2, 2, 2, g.K, g.Co, g.K, M, M, g.Co, 1, g.K, g.Co, 1, 0, 0};
            ops.matmul(g.K * g.Co, mm, cols, grad_flat, grad_w);
        }
        if (grad_bias) bias_gradient(ops, g, es, grad_out, sums, grad_bias);
        return;
    }
    char* grad_cols = ws;
    char* gw_batch = grad_cols + round16(g.B * g.K * g.P) * es;
    char* sums = gw_batch + round16(g.B * g.Co * g.K) * es;
    if (grad_x) {
        // grad_cols[B, K, P] = W^T (the transposed view of [Co, K], shared by every batch) . grad_out[B, Co, P]
        const size_t mm[20] = {3, 3, 3, g.B, g.K, g.P, g.B, g.K, g.Co, g.B, g.Co, g.P, 0, 1, g.K, g.Co * g.P, g.P, 1, 0, 0};
        ops.matmul(g.B * g.K * g.P, mm, w, grad_out, grad_cols);
        const size_t cm[12] = {g.B, g.C, g.H, g.W, g.kh, g.kw, g.oh, g.ow, g.ph, g.pw, g.sh, g.sw};
        ops.col2im(g.B * g.K * g.P, cm, grad_cols, grad_x);
    }
    if (grad_w) {
        // per batch grad_out[b][Co, P] . cols[b]^T (the transposed view of [K, P]), then the sum over the batch
        const size_t mm[20] = {3, 3, 3, g.B, g.Co, g.K, g.B, g.Co, g.P, g.B, g.P, g.K, g.Co * g.P, g.P, 1, g.K * g.P, 1, g.P, 0, 0};
        ops.matmul(g.B * g.Co * g.K, mm, grad_out, cols, gw_batch);
        const size_t d3[3] = {g.B, g.Co, g.K};
        sum_dim(ops, d3, 3, 0, gw_batch, grad_w);
    }
    if (grad_bias) bias_gradient(ops, g, es, grad_out, sums, grad_bias);
}

}  // namespace
}  // namespace mx

extern "C" {

size_t mx_conv2d_cols_elems(const MxConv2d* conv) {
    mx::Geometry g;
    return mx::geometry(conv, g) ? g.B * g.P * g.K : 0;
}
size_t mx_conv2d_output_elems(const MxConv2d* conv) {
    mx::Geometry g;
    return mx::geometry(conv, g) ? g.B * g.Co * g.P : 0;
}
size_t mx_conv2d_workspace_elems(const MxConv2d* conv, int mode, int backward) {
    mx::Geometry g;
    return mx::geometry(conv, g) ? mx::workspace_elems(g, mode, backward) : 0;
}

#define DEF_CONV2D(T)                                                                                                                   \
    void mx_conv2d_forward_##T(const MxConv2d* conv, int mode, const mx_##T* x, const mx_##T* weight, const mx_##T* bias, mx_##T* cols, \
                               mx_##T* workspace, mx_##T* out) {                                                                        \
        mx::forward(MX_CONV_OPS(T), sizeof(mx_##T), conv, mode, x, weight, bias, cols, workspace, out);                                 \
    }                                                                                                                                   \
    void mx_conv2d_backward_##T(const MxConv2d* conv, int mode, const mx_##T* grad_out, const mx_##T* weight, const mx_##T* cols,       \
                                mx_##T* workspace, mx_##T* grad_x, mx_##T* grad_weight, mx_##T* grad_bias) {                            \
        mx::backward(MX_CONV_OPS(T), sizeof(mx_##T), conv, mode, grad_out, weight, cols, workspace, grad_x, grad_weight, grad_bias);    \
    }
DEF_CONV2D(bf16)
DEF_CONV2D(f16)
DEF_CONV2D(f32)
DEF_CONV2D(f64)

}  // extern "C"
