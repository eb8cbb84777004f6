/*
 * maidenx_cuda.h — C ABI of the sm_100a op library (libmaidenx_cuda.so).
 *
 * Every `cuda_<op>_<dtype>` entry point below has the name, argument order and argument
 * meaning of the symbol of the same name that the reference's `maidenx_cuda` crate
 * declares for its own kernels and that `maidenx_core`'s backend dispatch calls; the
 * library is a link-time replacement for that crate's `libops.a` / `libnn.a`.
 *
 * Conventions shared by all op entry points (reference: crates/maidenx_cuda/src/ops/*.rs,
 * crates/maidenx_core/src/be/ops/binary.rs:96-169):
 *   - data pointers are device buffer BASE pointers; element offsets travel in `metadata`;
 *   - `metadata` is an array of size_t.  The reference uploads it to device memory before
 *     each call; this library accepts device memory (resolved through its upload wrappers
 *     without a device round trip, or read back when uploaded some other way) and, as an
 *     extension, plain host memory;
 *   - outputs are written contiguously from element 0 and never need to be pre-zeroed;
 *   - launches go to the legacy default stream of the calling thread's current device
 *     unless mx_set_stream() was called on that thread;
 *   - functions return void; failures are recorded in a sticky per-thread status
 *     (mx_last_error) instead of being silently dropped.
 *   - bf16 / f16 values cross the boundary as 16-bit patterns (the reference's half::bf16 /
 *     half::f16 are repr(transparent) u16), bool as one byte holding 0 or 1.
 */
#ifndef MAIDENX_CUDA_H
#define MAIDENX_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
typedef bool mx_bool;
#else
typedef _Bool mx_bool;
/* The dtype suffix `bool` is pasted into symbol names below; keep <stdbool.h>'s macro of
 * the same name out of the way while the declarations are generated. */
#pragma push_macro("bool")
#undef bool
#endif

/* Element types as they appear in pointer arguments.  When the library itself is built
 * the 16-bit float pointers are the CUDA vector types; callers see uint16_t. */
#ifdef MAIDENX_CUDA_BUILD
typedef __nv_bfloat16 mx_bf16;
typedef __half mx_f16;
#else
typedef uint16_t mx_bf16;
typedef uint16_t mx_f16;
#endif
typedef float mx_f32;
typedef double mx_f64;
typedef uint8_t mx_u8;
typedef uint16_t mx_u16;
typedef uint32_t mx_u32;
typedef uint64_t mx_u64;
typedef int8_t mx_i8;
typedef int16_t mx_i16;
typedef int32_t mx_i32;
typedef int64_t mx_i64;
/* By-value scalar arguments: 16-bit floats are passed as their bit pattern. */
typedef uint16_t mx_bf16_arg;
typedef uint16_t mx_f16_arg;
typedef float mx_f32_arg;
typedef double mx_f64_arg;
typedef mx_bool mx_bool_arg;
typedef uint8_t mx_u8_arg;
typedef uint16_t mx_u16_arg;
typedef uint32_t mx_u32_arg;
typedef uint64_t mx_u64_arg;
typedef int8_t mx_i8_arg;
typedef int16_t mx_i16_arg;
typedef int32_t mx_i32_arg;
typedef int64_t mx_i64_arg;

/* ---- dtype lists (X-macros: X(suffix, ...)) ------------------------------------------ */
#define MX_DTYPES_FLOAT(X, ...) X(bf16, __VA_ARGS__) X(f16, __VA_ARGS__) X(f32, __VA_ARGS__) X(f64, __VA_ARGS__)
#define MX_DTYPES_UINT(X, ...) X(u8, __VA_ARGS__) X(u16, __VA_ARGS__) X(u32, __VA_ARGS__) X(u64, __VA_ARGS__)
#define MX_DTYPES_SINT(X, ...) X(i8, __VA_ARGS__) X(i16, __VA_ARGS__) X(i32, __VA_ARGS__) X(i64, __VA_ARGS__)
#define MX_DTYPES_SIGNED(X, ...) MX_DTYPES_FLOAT(X, __VA_ARGS__) MX_DTYPES_SINT(X, __VA_ARGS__)
#define MX_DTYPES_ARITH(X, ...) MX_DTYPES_FLOAT(X, __VA_ARGS__) MX_DTYPES_UINT(X, __VA_ARGS__) MX_DTYPES_SINT(X, __VA_ARGS__)
#define MX_DTYPES_ALL(X, ...) MX_DTYPES_ARITH(X, __VA_ARGS__) X(bool, __VA_ARGS__)

/* ======================================================================================
 * Runtime wrappers — replace crates/maidenx_cuda/src/lib.rs:38-163 (`#[no_mangle] extern "C"`,
 * each returns the cudaError_t as int).  cuda_memcpy_h2d additionally records small uploads
 * so that metadata blocks can be resolved on the host; cuda_free forgets them.
 * ====================================================================================== */
typedef struct MxCudaPointerAttributes { /* lib.rs:23-29 */
    int type_;
    int device;
    void* devicePointer;
    void* hostPointer;
} MxCudaPointerAttributes;

int cuda_malloc(void** ptr, size_t size);                       /* lib.rs:38-41 */
int cuda_free(void* ptr);                                       /* lib.rs:47-50 */
int cuda_memcpy_h2d(void* dst, const void* src, size_t size);   /* lib.rs:58-61 */
int cuda_memcpy_d2h(void* dst, const void* src, size_t size);   /* lib.rs:69-72 */
int cuda_memcpy_d2d(void* dst, const void* src, size_t size);   /* lib.rs:80-83 */
int cuda_set_device(int device_id);                             /* lib.rs:107-110 */
int cuda_get_device(int* device_id);                            /* lib.rs:116-119 */
int cuda_stream_create(void** stream);                          /* lib.rs:125-128 */
int cuda_stream_destroy(void* stream);                          /* lib.rs:134-137 */
int cuda_stream_synchronize(void* stream);                      /* lib.rs:143-146 */
int cuda_pointer_get_attributes(MxCudaPointerAttributes* attributes, const void* ptr); /* lib.rs:153-163 */
const char* cuda_error_string(int error_code);                  /* C twin of the Rust-ABI cuda_error, lib.rs:90-100 */

/* ======================================================================================
 * Binary elementwise — replace crates/maidenx_cuda/src/ops/binary.rs:6-182
 * (kernels: crates/maidenx_cuda/kernels/ops/binary.cu:13-163; semantics follow the CPU
 * backend, crates/maidenx_cpu/src/ops/binary.rs:13-934).
 *   metadata = [dims(n) | lhs_strides(n) | rhs_strides(n) | lhs_offset, rhs_offset], or NULL
 *   out[i] = op(lhs[lhs_offset + idx_l(i)], rhs[rhs_offset + idx_r(i)])
 *   in-place: lhs[lhs_offset + idx_l(i)] = op(lhs[...], rhs[...])
 * dtype sets are the ones maidenx_core dispatches (crates/maidenx_core/src/be/ops/binary.rs:245-310).
 * ====================================================================================== */
#define MX_BINARY_ARITH_OPS(X, ...) X(add, __VA_ARGS__) X(sub, __VA_ARGS__) X(mul, __VA_ARGS__) X(div, __VA_ARGS__) X(maximum, __VA_ARGS__) X(minimum, __VA_ARGS__)
#define MX_BINARY_BOOL_OPS(X, ...) X(logical_and, __VA_ARGS__) X(logical_or, __VA_ARGS__) X(logical_xor, __VA_ARGS__) \
    X(eq, __VA_ARGS__) X(ne, __VA_ARGS__) X(lt, __VA_ARGS__) X(le, __VA_ARGS__) X(gt, __VA_ARGS__) X(ge, __VA_ARGS__)
#define MX_BINARY_INPLACE_OPS(X, ...) X(add_inplace, __VA_ARGS__) X(sub_inplace, __VA_ARGS__) X(mul_inplace, __VA_ARGS__) X(div_inplace, __VA_ARGS__)

#define MX_DECL_BINARY(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* lhs, const mx_##T* rhs, mx_##T* out);
#define MX_DECL_BINARY_BOOL(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* lhs, const mx_##T* rhs, mx_bool* out);
#define MX_DECL_BINARY_INPLACE(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, mx_##T* lhs, const mx_##T* rhs);
#define MX_DECL_BINARY_T(T, ...) MX_BINARY_ARITH_OPS(MX_DECL_BINARY, T) MX_BINARY_INPLACE_OPS(MX_DECL_BINARY_INPLACE, T)
#define MX_DECL_BINARY_BOOL_T(T, ...) MX_BINARY_BOOL_OPS(MX_DECL_BINARY_BOOL, T)
MX_DTYPES_ARITH(MX_DECL_BINARY_T, _)
MX_DTYPES_ALL(MX_DECL_BINARY_BOOL_T, _)

/* ======================================================================================
 * Unary elementwise — replace crates/maidenx_cuda/src/ops/unary.rs:6-192
 * (kernels: crates/maidenx_cuda/kernels/ops/unary.cu:9-88; CPU semantics:
 * crates/maidenx_cpu/src/ops/unary.rs:14-741).
 *   metadata = [dims(n) | strides(n) | offset], or NULL;  out[i] = op(in[offset + idx(i)][, constant])
 *   input == NULL means "read from out".
 * dtype sets: crates/maidenx_core/src/be/ops/unary.rs:486-526.
 * ====================================================================================== */
#define MX_UNARY_FLOAT_OPS(X, ...) X(relu, __VA_ARGS__) X(sigmoid, __VA_ARGS__) X(tanh, __VA_ARGS__) X(gelu, __VA_ARGS__) X(sin, __VA_ARGS__) \
    X(cos, __VA_ARGS__) X(tan, __VA_ARGS__) X(ln, __VA_ARGS__) X(log10, __VA_ARGS__) X(log2, __VA_ARGS__) X(exp, __VA_ARGS__)                \
    X(exp10, __VA_ARGS__) X(exp2, __VA_ARGS__) X(softplus, __VA_ARGS__) X(recip, __VA_ARGS__)
#define MX_UNARY_SIGNED_OPS(X, ...) X(neg, __VA_ARGS__) X(abs, __VA_ARGS__)
#define MX_UNARY_ARITH_OPS(X, ...) X(sign, __VA_ARGS__) X(square, __VA_ARGS__) X(sqrt, __VA_ARGS__)
#define MX_UNARY_CONST_ARITH_OPS(X, ...) X(add_scalar, __VA_ARGS__) X(sub_scalar, __VA_ARGS__) X(mul_scalar, __VA_ARGS__) X(div_scalar, __VA_ARGS__) \
    X(maximum_scalar, __VA_ARGS__) X(minimum_scalar, __VA_ARGS__) X(pow, __VA_ARGS__)
#define MX_UNARY_CONST_FLOAT_OPS(X, ...) X(leaky_relu, __VA_ARGS__) X(elu, __VA_ARGS__)
#define MX_UNARY_CONST_BOOL_OPS(X, ...) X(eq_scalar, __VA_ARGS__) X(ne_scalar, __VA_ARGS__) X(lt_scalar, __VA_ARGS__) X(le_scalar, __VA_ARGS__) \
    X(gt_scalar, __VA_ARGS__) X(ge_scalar, __VA_ARGS__)

#define MX_DECL_UNARY(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* input, mx_##T* output);
#define MX_DECL_UNARY_BOOL(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* input, mx_bool* output);
#define MX_DECL_UNARY_CONST(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* input, mx_##T##_arg constant, mx_##T* output);
#define MX_DECL_UNARY_CONST_BOOL(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* input, mx_##T##_arg constant, mx_bool* output);
#define MX_DECL_UNARY_FLOAT_T(T, ...) MX_UNARY_FLOAT_OPS(MX_DECL_UNARY, T) MX_UNARY_CONST_FLOAT_OPS(MX_DECL_UNARY_CONST, T)
#define MX_DECL_UNARY_SIGNED_T(T, ...) MX_UNARY_SIGNED_OPS(MX_DECL_UNARY, T)
#define MX_DECL_UNARY_ARITH_T(T, ...) MX_UNARY_ARITH_OPS(MX_DECL_UNARY, T) MX_UNARY_CONST_ARITH_OPS(MX_DECL_UNARY_CONST, T)
#define MX_DECL_UNARY_ALL_T(T, ...) MX_DECL_UNARY_BOOL(logical_not, T) MX_UNARY_CONST_BOOL_OPS(MX_DECL_UNARY_CONST_BOOL, T)
MX_DTYPES_FLOAT(MX_DECL_UNARY_FLOAT_T, _)
MX_DTYPES_SIGNED(MX_DECL_UNARY_SIGNED_T, _)
MX_DTYPES_ARITH(MX_DECL_UNARY_ARITH_T, _)
MX_DTYPES_ALL(MX_DECL_UNARY_ALL_T, _)

/* ======================================================================================
 * Reductions — replace crates/maidenx_cuda/src/ops/reduction.rs:6-104
 * (kernels: crates/maidenx_cuda/kernels/ops/reduction.cu:18-167,243-419; CPU semantics:
 * crates/maidenx_cpu/src/ops/reduction.rs:6-272,383-625).
 *   sum/mean/max/min: metadata = [dims(n) | strides(n) | red_len(r) | red_stride(r) | offset]
 *   sum_to_shape:     metadata = [in_dims(n) | in_strides(n) | out_dims(n) | offset]
 * The output is overwritten (no pre-zero contract); results are deterministic.
 * dtype sets: crates/maidenx_core/src/be/ops/reduction.rs:251-256.
 * ====================================================================================== */
#define MX_DECL_REDUCE(op, T) void cuda_##op##_##T(size_t num_els, size_t num_dims, size_t num_red_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out);
#define MX_DECL_REDUCE_ARITH_T(T, ...) MX_DECL_REDUCE(sum, T) MX_DECL_REDUCE(max, T) MX_DECL_REDUCE(min, T) \
    void cuda_sum_to_shape_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out);
#define MX_DECL_REDUCE_FLOAT_T(T, ...) MX_DECL_REDUCE(mean, T)
MX_DTYPES_ARITH(MX_DECL_REDUCE_ARITH_T, _)
MX_DTYPES_FLOAT(MX_DECL_REDUCE_FLOAT_T, _)

/* ======================================================================================
 * Matmul — replace crates/maidenx_cuda/src/ops/matmul.rs:6-50
 * (kernels: crates/maidenx_cuda/kernels/ops/matmul.cu:5-179; CPU semantics:
 * crates/maidenx_cpu/src/ops/matmul.rs:5-268).
 *   metadata = [out_ndim, a_ndim, b_ndim | out_shape | a_shape | b_shape | a_strides | b_strides | a_off, b_off]
 *   matmul:          C[b,m,n] = sum_k A[b,m,k] * B[b,k,n], C contiguous, num_els = batch*M*N
 *   matmul_backward: grad_a = g * B^T, grad_b = A^T * g with A, B, g read as contiguous
 *                    (strides ignored, offsets applied); either output may be NULL.
 * dtype set: crates/maidenx_core/src/be/ops/matmul.rs:265.
 * ====================================================================================== */
#define MX_DECL_MATMUL_T(T, ...)                                                                                                       \
    void cuda_matmul_##T(size_t num_els, const size_t* metadata, const mx_##T* a, const mx_##T* b, mx_##T* c);                        \
    void cuda_matmul_backward_##T(size_t num_els_a, size_t num_els_b, const size_t* metadata, const mx_##T* grad_output,               \
                                  const mx_##T* a, const mx_##T* b, mx_##T* grad_a, mx_##T* grad_b);
MX_DTYPES_ARITH(MX_DECL_MATMUL_T, _)

/* ======================================================================================
 * Conv2d helpers — replace crates/maidenx_cuda/src/nn/conv.rs:6-36
 * (kernels: crates/maidenx_cuda/kernels/nn/conv.cu:8-136; CPU semantics:
 * crates/maidenx_cpu/src/nn/conv.rs:13-149).
 *   metadata = [B, C, H, W, kh, kw, out_h, out_w, pad_h, pad_w, stride_h, stride_w]
 *   im2col: col[b][c,kh,kw][oh,ow] = x[b,c,oh*s-p+kh,ow*s-p+kw] or 0; num_els = col length
 *   col2im: every (b,c,h,w) is overwritten with the sum of the col entries mapping to it;
 *           num_els = readable length of col (entries beyond it are skipped).
 * dtype set: crates/maidenx_core/src/be/nn/conv.rs:240.
 * ====================================================================================== */
#define MX_DECL_CONV_T(T, ...)                                                                                     \
    void cuda_conv2d_im2col_##T(size_t num_els, const size_t* metadata, const mx_##T* input, mx_##T* col);        \
    void cuda_conv2d_col2im_##T(size_t num_els, const size_t* metadata, const mx_##T* col, mx_##T* output);
MX_DTYPES_FLOAT(MX_DECL_CONV_T, _)

/* ======================================================================================
 * fold, padding, softmax - the remaining families of the crate; generic kernels, not tuned
 * (declarations: crates/maidenx_cuda/src/ops/reduction.rs "fold", src/ops/padding.rs:6-91,
 * src/nn/activation/softmax.rs:6-31; CPU semantics: crates/maidenx_cpu/src/ops/reduction.rs:274-381,
 * src/ops/padding.rs, src/nn/activation/softmax.rs).
 *   fold:     metadata = [dims(n) | strides(n) | fold_dim, window_dim, fold_size, step, window_size, offset];
 *             out[.., w*step + p, ..] = sum of in[.., w, .., p, ..] (the backward of unfold); num_els = input elements
 *   padding:  metadata = [in_dims(n) | in_strides(n) | in_offset | out_dims(n) | (before, after) x n];
 *             forward (num_els_in, num_els_out, ..., inp, out[, pad_value]); backward (.., grad_out, grad_in) overwrites
 *             grad_in[in_offset .. in_offset + num_els_in) with the sums of the grad_out elements read from each position
 *   softmax:  metadata = [dims(n) | strides(n) | offset]; along `dim` (>= num_dims means the last); floats only
 * ====================================================================================== */
#define MX_DECL_EXTRA_ARITH_T(T, ...)                                                                                                              \
    void cuda_fold_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out);                                   \
    void cuda_pad_with_constant_##T(size_t num_els_in, size_t num_els_out, size_t num_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out, \
                                    mx_##T##_arg pad_value);                                                                                       \
    void cuda_pad_with_reflection_##T(size_t num_els_in, size_t num_els_out, size_t num_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out); \
    void cuda_pad_with_replication_##T(size_t num_els_in, size_t num_els_out, size_t num_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out); \
    void cuda_pad_with_constant_backward_##T(size_t num_els_in, size_t num_els_out, size_t num_dims, const size_t* metadata, const mx_##T* grad_out,  \
                                             mx_##T* grad_in);                                                                                     \
    void cuda_pad_with_reflection_backward_##T(size_t num_els_in, size_t num_els_out, size_t num_dims, const size_t* metadata, const mx_##T* grad_out, \
                                               mx_##T* grad_in);                                                                                   \
    void cuda_pad_with_replication_backward_##T(size_t num_els_in, size_t num_els_out, size_t num_dims, const size_t* metadata,                     \
                                                const mx_##T* grad_out, mx_##T* grad_in);
MX_DTYPES_ARITH(MX_DECL_EXTRA_ARITH_T, _)
#define MX_DECL_SOFTMAX_T(T, ...) \
    void cuda_softmax_##T(size_t num_els, size_t num_dims, size_t dim, const size_t* metadata, const mx_##T* input, mx_##T* output);
MX_DTYPES_FLOAT(MX_DECL_SOFTMAX_T, _)

/* ======================================================================================
 * Additive exports (no counterpart in the reference).
 * ====================================================================================== */
/* Tensor::contiguous() on the device: out[i] = in[offset + strided_index(i)], out dense.  The reference copies a
 * non-contiguous CUDA tensor to the host, walks it element by element and copies it back
 * (crates/maidenx_tensor/src/f.rs:11-40); this is the same gather in one launch, through the elementwise
 * engine (transposed views go through the tiled kernel).  metadata = [dims(n) | strides(n) | offset]. */
#define MX_DECL_CONTIGUOUS_T(T, ...) void mx_contiguous_##T(size_t num_els, size_t num_dims, const size_t* metadata, const mx_##T* inp, mx_##T* out);
MX_DTYPES_ALL(MX_DECL_CONTIGUOUS_T, _)

/* Dtype casts on the device, dense buffers: out[i] = cast(in[i]) with the element rules of the reference's host-side
 * conversion (crates/maidenx_core/src/buffer/mod.rs:132-575; listed in maidenx_b200/csrc/cast.cu).  One symbol per
 * ordered pair of the 13 dtypes: mx_cast_<from>_<to>(num_els, in, out). */
#define MX_CAST_TARGETS(X, FROM)                                                                                     \
    X(bf16, FROM) X(f16, FROM) X(f32, FROM) X(f64, FROM) X(bool, FROM) X(u8, FROM) X(u16, FROM) X(u32, FROM) X(u64, FROM) \
    X(i8, FROM) X(i16, FROM) X(i32, FROM) X(i64, FROM)
#define MX_DECL_CAST(TO, FROM) void mx_cast_##FROM##_##TO(size_t num_els, const mx_##FROM* in, mx_##TO* out);
#define MX_DECL_CAST_FROM(FROM, ...) MX_CAST_TARGETS(MX_DECL_CAST, FROM)
MX_DTYPES_ALL(MX_DECL_CAST_FROM, _)

/* cuda_malloc / cuda_free keep a cache: requests of up to 64 MB are rounded up to a size class (2 KB slots for the
 * per-call metadata blocks of the dispatch layer, powers of two above) and freed blocks go back to their class's
 * free list without the device synchronisation of cudaFree (at most 2 GB per device stay cached).  A block freed by a
 * thread that launches on its own stream (mx_set_stream) is handed out again only after the work queued on that
 * stream at the time of the free has finished.  Uploads of up to 2 KB through cuda_memcpy_h2d are staged in pinned
 * memory and copied asynchronously on the calling thread's current stream (the source is consumed before the call
 * returns; later work of the thread is ordered after the upload), so an op call no longer waits for the device.
 * 0 turns both off: every request goes to cudaMalloc / cudaFree / cudaMemcpy, as in the reference. */
void mx_set_small_pool(int enabled);

/* Stream used by this thread's subsequent op launches (NULL = legacy default stream). */
void mx_set_stream(void* stream);
void* mx_get_stream(void);
/* Sticky per-thread status: 0 = ok, 1 = CUDA error (see mx_last_cuda_error), 2 = bad metadata,
 * 3 = unsupported shape, 4 = no device, 5 = a bounded device-side wait ran out. */
int mx_last_error(void);
int mx_last_cuda_error(void);
const char* mx_last_error_where(void);
void mx_clear_error(void);
int mx_device_synchronize(void);
/* 0, or the wait that gave up in the last kernel of this thread's device that waits on copies it queued: tensor-core
 * matmuls (1 producer, 2/3 MMA issuer, 4 epilogue, ...), and the kernels fed through shared memory by the copy engine
 * (21 flat elementwise with staged operands, 22 transposed tiles of 2-byte types, 23 staged col2im).  A non-zero
 * value is also recorded as status 5.  Call after a synchronisation; cuda_memcpy_d2h and cuda_stream_synchronize
 * check it themselves and return non-zero. */
int mx_tc_gemm_status(void);
/* Number of metadata blocks currently remembered by cuda_memcpy_h2d (diagnostics). */
int mx_metadata_table_size(void);

/* cuda_sum_f32 for callers that must not allocate (in a latency-critical loop that has to stay free of
 * driver allocation calls, with all device memory owned by their own allocator, or where the allocating
 * runtime calls are not permitted).  No counterpart in the reference.
 * Same arguments as cuda_sum_f32 except that `metadata` must be host memory.  The second-pass
 * workspace is a fixed 1 MiB array inside the library (held on every GPU that loads it); a reduction
 * whose partials do not fit is rejected with status 3 and leaves `out` untouched.  The first call on
 * a device does the set-up (address of the array, SM count, occupancy) and should come before any stream
 * capture; calls share the
 * array, so calls that overlap on one GPU race.  Details: maidenx_b200/csrc/noalloc.cu. */
void mx_sum_f32_noalloc(size_t num_els, size_t num_dims, size_t num_red_dims, const size_t* metadata, const mx_f32* inp, mx_f32* out);

/* ---- fused elementwise passes of the training step (bf16, f16, f32) --------------------------
 * Each stands for a chain of single-op calls the reference's autograd issues; formulas and the
 * reference lines they follow are in maidenx_b200/csrc/fused.cu.  All pointers are device memory,
 * 16-byte aligned; `bias` is one element. */
#define MX_DECL_FUSED_T(T, ...)                                                                                         \
    void mx_bias_gelu_##T(size_t n, const mx_##T* z, const mx_##T* bias, mx_##T* u, mx_##T* a /* may be NULL */);        \
    void mx_gelu_backward_##T(size_t n, const mx_##T* dy, const mx_##T* u, mx_##T* du);                                  \
    void mx_mse_loss_grad_##T(size_t n, const mx_##T* pred, const mx_##T* target, mx_##T* grad, float* loss);            \
    void mx_sgd_update_##T(size_t n, float* w32, const mx_##T* grad, mx_##T* w16, float lr, float grad_scale);
MX_DECL_FUSED_T(bf16, _)
MX_DECL_FUSED_T(f16, _)
MX_DECL_FUSED_T(f32, _)
/* Linear forward in one call: u[rows, out] = x[rows, in] . w[out, in]^T + bias (one element), act = gelu(u); act may be
 * NULL.  Large layers run the product on the tensor cores with the bias add and the activation in its epilogue; the
 * results are the bits of cuda_matmul, cuda_add and cuda_gelu applied one after the other
 * (crates/maidenx_nn/src/layers/linear.rs:60-81). */
void mx_linear_bias_gelu_bf16(size_t rows, size_t in_features, size_t out_features, const mx_bf16* x, const mx_bf16* w, const mx_bf16* bias,
                              mx_bf16* u, mx_bf16* act);
void mx_linear_bias_gelu_f16(size_t rows, size_t in_features, size_t out_features, const mx_f16* x, const mx_f16* w, const mx_f16* bias,
                             mx_f16* u, mx_f16* act);

/* ---- Conv2d forward / backward composed from the ops above (maidenx_b200/csrc/conv2d_layer.cu) ---------------
 * The call sequence of the reference's layer (crates/maidenx_nn/src/layers/conv.rs:185-307,333-420): im2col,
 * matmul, bias add; backward: matmul + col2im (input gradient), matmul (weight gradient), three sums (bias
 * gradient).  mode 0 issues exactly the calls the reference's layer issues (column buffer declared [B*oh*ow, K],
 * stride/padding slot order, col2im with num_els = B*C*H*W); mode 1 uses the same ops consistently (batched
 * product with the weight shared by every batch) and is a true convolution.  x [B, C, H, W], weight
 * [Cout, C, kh, kw], bias [Cout] or NULL, out / grad_out [B, Cout, oh, ow], all dense; `cols` has
 * mx_conv2d_cols_elems elements and carries im2col's result from forward to backward; `workspace` has
 * mx_conv2d_workspace_elems(conv, mode, backward) elements.  Any of grad_x / grad_weight / grad_bias may be NULL.
 * In mode 0 grad_weight is the [C*kh*kw, Cout] product the reference re-labels as [Cout, C, kh, kw]. */
typedef struct MxConv2d {
    size_t batch, in_channels, height, width, out_channels, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w;
} MxConv2d;
size_t mx_conv2d_cols_elems(const MxConv2d* conv);
size_t mx_conv2d_output_elems(const MxConv2d* conv);
size_t mx_conv2d_workspace_elems(const MxConv2d* conv, int mode, int backward);
#define MX_DECL_CONV2D_T(T, ...)                                                                                                        \
    void mx_conv2d_forward_##T(const MxConv2d* conv, int mode, const mx_##T* x, const mx_##T* weight, const mx_##T* bias, mx_##T* cols, \
                               mx_##T* workspace, mx_##T* out);                                                                         \
    void mx_conv2d_backward_##T(const MxConv2d* conv, int mode, const mx_##T* grad_out, const mx_##T* weight, const mx_##T* cols,       \
                                mx_##T* workspace, mx_##T* grad_x, mx_##T* grad_weight, mx_##T* grad_bias);
MX_DTYPES_FLOAT(MX_DECL_CONV2D_T, _)

/* ---- MLP training step (the data-parallel workload; maidenx_b200/csrc/mlp.cu) ------------------
 * L x [Linear(dim -> dim) + scalar bias, GELU between layers], MSE, SGD with f32 master weights.
 * dtype: 0 = bf16, 1 = f16.  x, y: [batch, dim] device buffers.  The step is forward,
 * loss_backward, then backward_layer(l) for l = L-1 .. 0 and sgd_layer(l); a data-parallel driver
 * all-reduces mx_mlp_weight_grad(l) / mx_mlp_bias_grad(l) between the last two. */
void* mx_mlp_create(int layers, size_t dim, size_t batch, int dtype, uint64_t seed);
void mx_mlp_destroy(void* mlp);
void mx_mlp_forward(void* mlp, const void* x);
void mx_mlp_loss_backward(void* mlp, const void* y);
void mx_mlp_backward_layer(void* mlp, int layer);
void mx_mlp_sgd_layer(void* mlp, int layer, float lr, float grad_scale);
/* forward, loss, backward and the optimizer update of every layer in one call (single-device engine); the updates run
 * on a side stream beside the backward of the layers below.  mx_mlp_dp_join makes the calling thread's stream wait for
 * them (the next mx_mlp_train_step / mx_mlp_forward waits by itself). */
void mx_mlp_train_step(void* mlp, const void* x, const void* y, float lr, float grad_scale);
void* mx_mlp_weight_grad(void* mlp, int layer);
void* mx_mlp_bias_grad(void* mlp, int layer);
float* mx_mlp_master_weight(void* mlp, int layer);
float* mx_mlp_master_bias(void* mlp, int layer);
void* mx_mlp_weight(void* mlp, int layer);
void* mx_mlp_output(void* mlp);
float* mx_mlp_loss_ptr(void* mlp);
float mx_mlp_loss(void* mlp);

/* ---- data-parallel exchange fused with the SGD step, over NVLink (maidenx_b200/csrc/dp_sync.cu) --
 * No counterpart in the reference, which trains on one device; the per-rank arithmetic is its
 * SGD step (crates/maidenx_nn/src/optimizers/sgd.rs:17-26) applied to the summed gradient.
 * Every rank provides an "arena" that is mapped into all ranks (peer pointers) and optionally bound
 * to a multicast address; the library never allocates or exchanges it.
 *   mx_dp_barrier      flag barrier across ranks, queued on `stream` (NULL: the thread's stream);
 *                      peer_arenas[p] + flag_offset = `world` zero-initialised u32 flags in rank p's
 *                      arena; `epoch` grows by one per barrier; a wait gives up after about two
 *                      seconds and stores 1 + peer in *err (device word).
 *   mx_dp_reduce_sgd   this rank's shard of one layer: g = sum over ranks of the gradient at
 *                      grad_offset (multimem.ld_reduce through multicast_arena, or peer loads when
 *                      it is NULL); master_shard -= step * g; the rounded weights are written to
 *                      weight_offset of EVERY arena (multimem.st or peer stores).  The scalar bias
 *                      (gradient slot at bias_grad_offset) is updated by every rank.  dtype 0 = bf16,
 *                      1 = f16; shard_begin and shard_elems count elements and are multiples of 8.
 *                      staged_grads != NULL: the peers' gradient shards were copied to local memory
 *                      (copy engines) and the weights are written to the local arena only; the caller
 *                      copies them to the peers.  exclusive_sms = k > 0 (multicast form): k blocks of
 *                      1024 threads that share their SMs with no GEMM block.
 * mx_mlp_create_dp / mx_mlp_train_step_dp run the MLP step on top of these: gradients and 16-bit
 * weights live in the arena (mx_mlp_dp_arena_bytes, zero-filled, 4 KiB aligned), `batch` is the
 * rank's share, and each layer's exchange overlaps the backward of the layers below it.
 * mx_mlp_dp_join makes the calling thread's stream wait for the exchange of the last step;
 * mx_mlp_dp_status waits on the host and returns 0 or 1 + the peer a barrier gave up on. */
void mx_dp_barrier(void* const* peer_arenas, size_t flag_offset, int rank, int world, uint32_t epoch, uint32_t* err, void* stream);
void mx_dp_reduce_sgd(int dtype, void* const* peer_arenas, void* multicast_arena, const void* const* staged_grads, int rank, int world,
                      size_t grad_offset, size_t weight_offset, size_t bias_grad_offset, float* master_shard, size_t shard_begin, size_t shard_elems,
                      float* master_bias, void* bias16, float step, int exclusive_sms, void* stream);
size_t mx_mlp_dp_arena_bytes(int layers, size_t dim);
void* mx_mlp_create_dp(int layers, size_t dim, size_t batch, int dtype, uint64_t seed, int rank, int world, void* const* peer_arenas,
                       void* multicast_arena);
void mx_mlp_train_step_dp(void* mlp, const void* x, const void* y, float lr, float grad_scale);
uint32_t mx_mlp_dp_status(void* mlp);
void mx_mlp_dp_join(void* mlp);
/* mode 0: the exchange runs in the library's NVLink kernel (multimem or peer form); exclusive_sms = k > 0 runs the
 * multimem form as k blocks that keep k SMs to themselves while every GEMM of the step uses the others.
 * mode 1: transfers by device-to-device copies (copy engines), sum and update in a local kernel.  Returns 0 or -1. */
int mx_mlp_dp_set_exchange(void* mlp, int mode, int exclusive_sms);
/* The tensor-core GEMM of the calling thread launches at most `sms` CTAs (0: all SMs), leaving the other SMs to a
 * concurrent kernel such as the exchange above. */
void mx_set_gemm_sm_limit(int sms);
/* 1 (default): one CTA per output tile; 2: bf16 / f16 products on the tensor cores run as pairs of CTAs on neighbouring
 * SMs that share the B tile (tcgen05.mma.cta_group::2).  Same results and, on a power-capped B200, the same rate;
 * process-wide. */
void mx_set_gemm_cta_group(int ctas);

#ifdef __cplusplus
}
#else
#pragma pop_macro("bool")
#endif
#endif /* MAIDENX_CUDA_H */
