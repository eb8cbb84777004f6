// conv2d im2col / col2im for one dtype (MX_T).
// Replaces the symbols declared in crates/maidenx_cuda/src/nn/conv.rs:6-36; semantics follow
// crates/maidenx_cpu/src/nn/conv.rs:13-149.
//   metadata = [B, C, H, W, kh, kw, out_h, out_w, pad_h, pad_w, stride_h, stride_w]
//   col layout [B][C, kh, kw][out_h, out_w]
//
// im2col: one block per (b, c) image plane.  The plane is read once into shared memory
// with coalesced loads; each of the kh*kw shifted copies is then written as one contiguous
// run of out_h*out_w elements with 16-byte stores.  DRAM traffic is the algorithmic
// minimum (input once + col once) where the reference re-reads the input kh*kw times.
//
// col2im: gather formulation, one thread per output pixel summing the (at most kh*kw) col
// entries that map to it in the reference's (h_out, w_out) order and in the element type,
// so the result is bit-identical to the CPU backend, deterministic, needs no atomics and
// overwrites the output (the reference's CUDA kernel scatters with atomicAdd into a
// pre-zeroed buffer).  `num_els` bounds the readable part of col: entries at or beyond it
// are skipped, as the CPU backend does (conv.rs:135).
#include "abi_common.cuh"
#include "conv_s1.cuh"
#include "ops.cuh"

#ifndef MX_T
#error "compile with -DMX_T=<dtype suffix> -DMX_TCLASS=<class>"
#endif

namespace mx {

struct ConvParams {
    uint32_t B, C, H, W, KH, KW, OH, OW, PH, PW, SH, SW;
    uint64_t num_els;
    FastDiv ow_div, w_div;
};

constexpr int kConvThreads = 256;

template <class T, int VEC, bool STAGED>
__global__ void __launch_bounds__(kConvThreads) im2col_kernel(const T* __restrict__ x, T* __restrict__ col, ConvParams P) {
    extern __shared__ __align__(16) unsigned char conv_smem[];
    T* plane = reinterpret_cast<T*>(conv_smem);
    const uint64_t bc = blockIdx.x;  // b * C + c
    const uint32_t HW = P.H * P.W, OHW = P.OH * P.OW, KK = P.KH * P.KW;
    const T* src = x + bc * HW;
    if constexpr (STAGED) {
        for (uint32_t i = threadIdx.x; i < HW; i += kConvThreads) plane[i] = src[i];
        __syncthreads();
    }
    const T* img = STAGED ? plane : src;
    const T zero = zero_of<T>();
    const uint64_t out_base = bc * KK * OHW;
    const uint32_t nvec = (OHW + VEC - 1) / VEC;
    for (uint32_t kk = 0; kk < KK; kk++) {
        const uint32_t kh = kk / P.KW, kw = kk % P.KW;
        T* dst = col + out_base + (uint64_t)kk * OHW;
        const uint64_t dst_lin = out_base + (uint64_t)kk * OHW;
        for (uint32_t v = threadIdx.x; v < nvec; v += kConvThreads) {
            Vec<T, VEC> r;
            uint32_t o0 = v * VEC;
            uint32_t ho, wo;
            P.ow_div.divmod(o0, ho, wo);
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                int hi = (int)(ho * P.SH + kh) - (int)P.PH, wi = (int)(wo * P.SW + kw) - (int)P.PW;
                bool in = hi >= 0 && hi < (int)P.H && wi >= 0 && wi < (int)P.W && o0 + j < OHW;
                r.v[j] = in ? img[hi * P.W + wi] : zero;
                if (++wo == P.OW) {
                    wo = 0;
                    ho++;
                }
            }
            if (VEC > 1 && o0 + VEC <= OHW && dst_lin + o0 + VEC <= P.num_els) {
                *reinterpret_cast<Vec<T, VEC>*>(dst + o0) = r;
            } else {
#pragma unroll
                for (int j = 0; j < VEC; j++)
                    if (o0 + j < OHW && dst_lin + o0 + j < P.num_els) dst[o0 + j] = r.v[j];
            }
        }
    }
}

template <class T>
__device__ __forceinline__ T conv_add(T a, T b) {
    if constexpr (is_half_v<T>) return from_f32<T>(to_f32(a) + to_f32(b));
    else return a + b;
}

template <class T>
__global__ void __launch_bounds__(kConvThreads) col2im_kernel(const T* __restrict__ col, T* __restrict__ out, ConvParams P) {
    const uint64_t bc = blockIdx.y;  // b * C + c
    const uint32_t HW = P.H * P.W, OHW = P.OH * P.OW, KK = P.KH * P.KW;
    const uint32_t pix = blockIdx.x * kConvThreads + threadIdx.x;
    if (pix >= HW) return;
    uint32_t h, w;
    P.w_div.divmod(pix, h, w);
    const uint32_t hp = h + P.PH, wp = w + P.PW;
    // conv.rs:121-125
    const uint32_t hs0 = hp >= P.KH - 1 ? hp - (P.KH - 1) : 0, ws0 = wp >= P.KW - 1 ? wp - (P.KW - 1) : 0;
    const uint32_t hs = (hs0 + P.SH - 1) / P.SH, ws = (ws0 + P.SW - 1) / P.SW;
    const uint32_t he = min(hp / P.SH + 1, P.OH), we = min(wp / P.SW + 1, P.OW);
    const uint64_t base = bc * KK * OHW;
    T sum = zero_of<T>();
    for (uint32_t ho = hs; ho < he; ho++) {
        const uint32_t kh = hp - ho * P.SH;
        if (kh >= P.KH) continue;
        for (uint32_t wo = ws; wo < we; wo++) {
            const uint32_t kw = wp - wo * P.SW;
            if (kw >= P.KW) continue;
            uint64_t ci = base + (uint64_t)(kh * P.KW + kw) * OHW + ho * P.OW + wo;
            if (ci < P.num_els) sum = conv_add(sum, col[ci]);
        }
    }
    out[bc * HW + pix] = sum;
}

static bool conv_params(const size_t* meta, size_t num_els, ConvParams& P, const char* where) {
    const size_t* m = resolve_metadata(meta, 12);
    if (!m) return false;
    for (int i = 0; i < 12; i++)
        if (m[i] > 0x7FFFFFFFull) {
            set_error(kErrUnsupported, 0, where);
            return false;
        }
    P.B = (uint32_t)m[0];
    P.C = (uint32_t)m[1];
    P.H = (uint32_t)m[2];
    P.W = (uint32_t)m[3];
    P.KH = (uint32_t)m[4];
    P.KW = (uint32_t)m[5];
    P.OH = (uint32_t)m[6];
    P.OW = (uint32_t)m[7];
    P.PH = (uint32_t)m[8];
    P.PW = (uint32_t)m[9];
    P.SH = (uint32_t)m[10];
    P.SW = (uint32_t)m[11];
    P.num_els = num_els;
    if (P.SH == 0 || P.SW == 0) {  // division by zero in the reference's index arithmetic
        set_error(kErrBadMetadata, 0, where);
        return false;
    }
    P.ow_div.init(P.OW);
    P.w_div.init(P.W);
    return true;
}

template <class T>
void im2col_entry(size_t num_els, const size_t* meta, const T* x, T* col, const char* where) {
    if (!meta || !x || !col) return;  // conv.rs:19-21
    ConvParams P;
    if (!conv_params(meta, num_els, P, where)) return;
    const uint64_t planes = (uint64_t)P.B * P.C;
    const uint64_t chunk = (uint64_t)P.KH * P.KW * P.OH * P.OW;
    if (planes == 0 || chunk == 0 || num_els == 0) return;
    // the reference walks col in chunks of C*kh*kw*oh*ow per batch; planes beyond num_els are never touched
    uint64_t planes_touched = (num_els + chunk - 1) / chunk;
    if (planes_touched > planes) planes_touched = planes;
    if (planes_touched > 0x7FFFFFFFull) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    constexpr int VEC = 16 / sizeof(T);
    const size_t plane_bytes = (size_t)P.H * P.W * sizeof(T);
    const bool vec = ((uintptr_t)col % 16 == 0) && ((uint64_t)P.OH * P.OW) % VEC == 0;
    cudaStream_t s = ctx().stream;
    const unsigned grid = (unsigned)planes_touched;
    // stride-1 fast path (conv_s1.cuh)
    if (P.SH == 1 && P.SW == 1 && vec && P.OW % VEC == 0 && num_els == planes * chunk && (int)P.KW - 1 <= VEC &&
        (uint64_t)P.OW + P.KW == (uint64_t)P.W + 2 * P.PW + 1 && (uint64_t)P.OH + P.KH == (uint64_t)P.H + 2 * P.PH + 1) {
        ConvS1Params Q;
        Q.H = P.H; Q.W = P.W; Q.KH = P.KH; Q.OH = P.OH; Q.OW = P.OW; Q.PH = P.PH; Q.PW = P.PW;
        Q.owv = P.OW / VEC;
        uint32_t need = (Q.owv + 1) * VEC, wide = (P.W + 2 * P.PW + VEC - 1) / VEC * VEC;
        Q.pitch = need > wide ? need : wide;
        Q.num_els = num_els;
        const size_t smem = (size_t)(P.H + 2 * P.PH) * Q.pitch * sizeof(T);
        auto go = [&](auto kernel) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            kernel<<<grid, kConvS1Threads, smem, s>>>(x, col, Q);
            check_launch(where);
        };
        if (smem <= 200 * 1024) {
            switch (P.KW) {
                case 1: go(im2col_s1_kernel<T, VEC, 1>); return;
                case 3: if (VEC >= 2) { go(im2col_s1_kernel<T, VEC, 3>); return; } break;
                case 5: if (VEC >= 4) { go(im2col_s1_kernel<T, VEC, 5>); return; } break;
                case 7: if (VEC >= 8) { go(im2col_s1_kernel<T, VEC, 7>); return; } break;
                default: break;
            }
        }
    }
    if (plane_bytes <= 200 * 1024) {
        auto launch = [&](auto kernel) {
            if (plane_bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plane_bytes);
            kernel<<<grid, kConvThreads, plane_bytes, s>>>(x, col, P);
        };
        if (vec) launch(im2col_kernel<T, VEC, true>);
        else launch(im2col_kernel<T, 1, true>);
    } else {
        if (vec) im2col_kernel<T, VEC, false><<<grid, kConvThreads, 0, s>>>(x, col, P);
        else im2col_kernel<T, 1, false><<<grid, kConvThreads, 0, s>>>(x, col, P);
    }
    check_launch(where);
}

template <class T>
void col2im_entry(size_t num_els, const size_t* meta, const T* col, T* out, const char* where) {
    if (!meta || !col || !out) return;  // conv.rs:90-92
    ConvParams P;
    if (!conv_params(meta, num_els, P, where)) return;
    const uint64_t planes = (uint64_t)P.B * P.C, HW = (uint64_t)P.H * P.W;
    if (planes == 0 || HW == 0) return;
    if (planes > 65535ull * 65535ull || P.KH == 0 || P.KW == 0) {
        set_error(kErrUnsupported, 0, where);
        return;
    }
    cudaStream_t s = ctx().stream;
    // stride-1 fast path (conv_s1.cuh)
    {
        constexpr int VEC = 16 / sizeof(T);
        const int kw = (int)P.KW, pw = (int)P.PW;
        const bool shape_ok = P.SH == 1 && P.SW == 1 && P.W % VEC == 0 && P.OW % VEC == 0 && num_els % VEC == 0 &&
                              ((uintptr_t)col | (uintptr_t)out) % 16 == 0 && planes <= 65535 && pw < VEC && kw - 1 - pw < VEC && kw - 1 - pw >= 0 &&
                              (uint64_t)P.OW + P.KW == (uint64_t)P.W + 2 * P.PW + 1 && (uint64_t)P.OH + P.KH == (uint64_t)P.H + 2 * P.PH + 1;
        if (shape_ok) {
            ConvS1Params Q;
            Q.H = P.H; Q.W = P.W; Q.KH = P.KH; Q.OH = P.OH; Q.OW = P.OW; Q.PH = P.PH; Q.PW = P.PW;
            Q.pitch = 0;
            Q.owv = P.OW / VEC;
            Q.num_els = num_els;
            const uint32_t items = P.H * (P.W / VEC);
            dim3 grid((items + kConvS1Threads - 1) / kConvS1Threads, (unsigned)planes);
            // every plane readable, 16-byte-multiple planes, at least two blocks' worth of shared memory per SM: staged form
            const uint64_t plane_elems = (uint64_t)P.KH * P.KW * P.OH * P.OW;
            const size_t stage_bytes = (size_t)plane_elems * sizeof(T);
            if (num_els >= planes * plane_elems && stage_bytes % 16 == 0 && stage_bytes <= 112 * 1024 && plane_elems < (1ull << 30)) {
                auto go = [&](auto kernel) {
                    if (stage_bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage_bytes);
                    kernel<<<(unsigned)planes, kConvS1Threads, stage_bytes, s>>>(col, out, Q, tc::next_wait_report());
                    check_launch(where);
                };
                if (kw == 1 && pw == 0) { go(col2im_s1_staged_kernel<T, VEC, 1, 0>); return; }
                if (kw == 3 && pw == 1) { go(col2im_s1_staged_kernel<T, VEC, 3, 1>); return; }
                if (kw == 3 && pw == 0 && VEC > 2) { go(col2im_s1_staged_kernel<T, VEC, 3, 0>); return; }
                if (kw == 5 && pw == 2 && VEC > 2) { go(col2im_s1_staged_kernel<T, VEC, 5, 2>); return; }
                if (kw == 7 && pw == 3 && VEC > 3) { go(col2im_s1_staged_kernel<T, VEC, 7, 3>); return; }
            }
            bool done = true;
            if (kw == 1 && pw == 0) col2im_s1_kernel<T, VEC, 1, 0><<<grid, kConvS1Threads, 0, s>>>(col, out, Q);
            else if (kw == 3 && pw == 1) col2im_s1_kernel<T, VEC, 3, 1><<<grid, kConvS1Threads, 0, s>>>(col, out, Q);
            else if (kw == 3 && pw == 0 && VEC > 2) col2im_s1_kernel<T, VEC, 3, 0><<<grid, kConvS1Threads, 0, s>>>(col, out, Q);
            else if (kw == 5 && pw == 2 && VEC > 2) col2im_s1_kernel<T, VEC, 5, 2><<<grid, kConvS1Threads, 0, s>>>(col, out, Q);
            else if (kw == 7 && pw == 3 && VEC > 3) col2im_s1_kernel<T, VEC, 7, 3><<<grid, kConvS1Threads, 0, s>>>(col, out, Q);
            else done = false;
            if (done) {
                check_launch(where);
                return;
            }
        }
    }
    // grid.y carries the plane index; fold very large plane counts into several launches
    const unsigned gx = (unsigned)((HW + kConvThreads - 1) / kConvThreads);
    for (uint64_t p0 = 0; p0 < planes; p0 += 65535) {
        uint64_t cnt = planes - p0 < 65535 ? planes - p0 : 65535;
        ConvParams Q = P;
        // shift the views instead of the plane index: col entries of plane p start at p*KK*OHW
        const uint64_t col_shift = p0 * P.KH * P.KW * P.OH * P.OW;
        Q.num_els = num_els > col_shift ? num_els - col_shift : 0;
        col2im_kernel<T><<<dim3(gx, (unsigned)cnt), kConvThreads, 0, s>>>(col + col_shift, out + p0 * HW, Q);
    }
    check_launch(where);
}

}  // namespace mx

#define DEF_CONV_(T)                                                                                          \
    void cuda_conv2d_im2col_##T(size_t n, const size_t* m, const mx_##T* i, mx_##T* o) {                      \
        mx::im2col_entry<mx_##T>(n, m, i, o, "cuda_conv2d_im2col_" #T);                                       \
    }                                                                                                         \
    void cuda_conv2d_col2im_##T(size_t n, const size_t* m, const mx_##T* i, mx_##T* o) {                      \
        mx::col2im_entry<mx_##T>(n, m, i, o, "cuda_conv2d_col2im_" #T);                                       \
    }
#define DEF_CONV(T) DEF_CONV_(T)

extern "C" {
DEF_CONV(MX_T)
}
