/* C ABI of the B200 implementation of the TP-invariant row-split path.
 *
 * One shared library (libtbik_b200.so) exports these entry points.  They take plain device
 * pointers, sizes and a CUDA stream; no torch types cross this boundary.  Every function
 * returns TBIK_OK (0) or a negative TBIK_ERR_* code and never throws; the message for the
 * last error of the calling thread is available from tbik_last_error().
 *
 * Each declaration names the reference interface it stands in for (paths are relative to the
 * reference project).
 */
#ifndef TBIK_H_
#define TBIK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ---------------------------------------------------------------------- */
#define TBIK_OK 0
#define TBIK_ERR_ARG (-1)    /* null pointer / bad handle / bad enum                         */
#define TBIK_ERR_SHAPE (-2)  /* sizes the path cannot take (K not a multiple of the leaf ...) */
#define TBIK_ERR_DTYPE (-3)  /* element type not supported                                    */
#define TBIK_ERR_ALIGN (-4)  /* pointer or stride alignment                                   */
#define TBIK_ERR_CUDA (-5)   /* a CUDA runtime / driver call failed                           */
#define TBIK_ERR_STATE (-6)  /* unregistered buffer, capacity exhausted, closed handle        */
#define TBIK_ERR_DEVICE (-7) /* a kernel gave up on a bounded wait and reported it            */

/* ---- element types --------------------------------------------------------------------- */
#define TBIK_DTYPE_BF16 0
#define TBIK_DTYPE_FP16 1
#define TBIK_DTYPE_FP32 2

/* Type of the tree nodes of the GEMM. */
#define TBIK_NODE_INPUT 0 /* nodes rounded to the operand type: the reference's arithmetic   */
#define TBIK_NODE_FP32 1  /* nodes kept in fp32, one final rounding                            */

typedef void* tbik_stream_t; /* a cudaStream_t */

/* Message of the last failing call made by this thread ("" if none). */
const char* tbik_last_error(void);

/* Library / ABI version: major * 1000 + minor. */
int tbik_version(void);

/* (T, F, L) of the reduction tree for a K extent and leaf width: T leaves, level 0 sums F
 * consecutive leaves, L levels in all (T = F * 2^(L-1)).
 * Replaces: src/tbik/tree_based_matmul.py:240-249 (TILE_K, FIRST_LEVEL_BLOCK, LEVEL_K). */
int tbik_tree_shape(int64_t K, int leaf, int* T, int* F, int* L);

/* C[M,N] = A[M,K] * W[N,K]^T with the K reduction done in the fixed tree order.
 *   A   row-major, row stride lda elements; W row-major [N,K] (the K-contiguous weight, i.e.
 *       the reference's B = weight.t() without the transpose), row stride ldw; C row stride ldc.
 *   dtype       TBIK_DTYPE_BF16 or TBIK_DTYPE_FP16 (operands and C)
 *   leaf        leaf width in elements, multiple of 64 (the reference uses 256)
 *   node_dtype  TBIK_NODE_INPUT
 * A and W must be 16-byte aligned with lda, ldw multiples of 8.  M == 0 or N == 0 is a no-op.
 * The kernel is enqueued on `stream`; it needs no workspace and allocates nothing.
 * Replaces: matmul_tp_persistent / matmul_kernel_tp_persistent,
 *           src/tbik/tree_based_matmul.py:50-187 and :190-274. */
int tbik_gemm(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
              int dtype, int leaf, int node_dtype, tbik_stream_t stream);

/* As tbik_gemm, but runs on at most `max_ctas` CTAs (0 = one per SM).  The result does not
 * depend on max_ctas; the entry point exists so that tests can prove that. */
int tbik_gemm_ex(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 int dtype, int leaf, int node_dtype, int max_ctas, tbik_stream_t stream);

/* Reads (and clears) the device-side status of the GEMM kernels on the current device:
 * out[0] != 0 means a kernel gave up on a bounded wait (out[1] = block, out[2] = role).
 * Synchronises with the device.  No counterpart in the reference (its waits are unbounded). */
int tbik_gemm_status(uint32_t out[4]);

#ifdef __cplusplus
}
#endif
#endif /* TBIK_H_ */
