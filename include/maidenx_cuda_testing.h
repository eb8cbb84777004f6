/* Test-only exports of libmaidenx_cuda.so: host-side views of the launch planners and hooks that let a test
 * reach a state it must not produce on a GPU.  Not part of the op layer's public interface (maidenx_cuda.h);
 * no counterpart in the reference. */
#ifndef MAIDENX_CUDA_TESTING_H
#define MAIDENX_CUDA_TESTING_H
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Host-only views of the launch planners, for tests that run without a GPU: which kernel class a call with this
 * HOST metadata and these base addresses would take.  Elementwise: 0 empty, 1 flat, 2 row, 3 tile, 4 generic,
 * 5 serial (an in-place lhs that overlaps itself), 6 error, 7 flat with shifted loads (operands not 16-byte aligned).  Reduction: 0 empty, 1 rows, 2 columns, 3 generic
 * scatter, 4 error, with the recognised [outer, reduced, inner] extents. */
int mx_debug_elementwise_plan(size_t num_els, size_t num_dims, const size_t* host_metadata, int num_inputs, int inplace, size_t elem_size,
                              size_t out_elem_size, const void* out, const void* a, const void* b, int* merged_rank, int* vector_ok,
                              int* transposed_mask);
/* Would cuda_matmul_<bf16|f16> with this HOST metadata run on the tcgen05 kernel (1) or on the SIMT kernel (0)?
 * Also returns the operand layouts (0 = K-major, 1 = MN-major) and the extents of the launch. */
int mx_debug_matmul_forward_path(size_t num_els, const size_t* host_metadata, const void* a, const void* b, const void* out, int* a_mn_major,
                                 int* b_mn_major, size_t* m, size_t* n, size_t* k);
int mx_debug_reduce_plan(size_t num_els, size_t num_dims, size_t num_red_dims, const size_t* host_metadata, int sum_to_shape, size_t* outer,
                         size_t* reduced, size_t* inner);

/* Would cuda_matmul_f32 with this HOST metadata run on the tcgen05 split-tf32 kernel (1) or on the SIMT kernel (0)? */
int mx_debug_matmul_forward_path_f32(size_t num_els, const size_t* host_metadata, const void* a, const void* b, const void* out, int* a_mn_major,
                                     int* b_mn_major, size_t* m, size_t* n, size_t* k);
/* Tuning aid: row-tiles per column sweep in the one-CTA tensor-core kernel's tile order (default 16). */
void mx_debug_set_gemm_group_m(int rows);
/* Pairs of CTAs of the two-CTA tensor-core kernel that can be resident at once on the current device (-1: query failed). */
int mx_debug_gemm_max_resident_pairs(void);
/* Short reductions (K <= 256, one batch, many row tiles) keep the B panel of a column tile in shared memory and stream
 * only A.  set: 1 = on (default), 0 = always the general schedule.  The query returns the CTAs per column tile a launch
 * with these tile counts takes (0 = general schedule). */
void mx_debug_set_gemm_keep_b(int on);
int mx_debug_gemm_keep_b_ctas(int tiles_m, int tiles_n, int num_kb, int batch, int ctas);
/* How many K slices the tensor-core path cuts a product with `tiles` output tiles and reduction length `k` into
 * (1 = no split) on `sms` SMs; block_k = 64 for bf16 / f16, 32 for f32. */
int mx_debug_splitk_slices(size_t tiles, size_t k, int block_k, int sms);
/* Writes `value` (0 clears) into the calling thread's tensor-core error word the way a kernel of an earlier launch
 * whose bounded wait ran out would have left it.  Returns 0, or -1 without a usable device. */
int mx_debug_tc_gemm_poke_status(int value);

#ifdef __cplusplus
}
#endif
#endif /* MAIDENX_CUDA_TESTING_H */
