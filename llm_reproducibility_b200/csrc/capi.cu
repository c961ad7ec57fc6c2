// extern "C" surface of libtbik_b200.so: argument plumbing and error strings only.
#include <stdio.h>
#include <string.h>

#include "tbik_internal.h"

namespace tbik {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char* msg) {
  snprintf(g_last_error, sizeof(g_last_error), "%s", msg ? msg : "");
  return code;
}

int set_cuda_error(cudaError_t e, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return TBIK_ERR_CUDA;
}

}  // namespace tbik

extern "C" {

const char* tbik_last_error(void) { return tbik::g_last_error; }

int tbik_version(void) { return 1000; }

int tbik_tree_shape(int64_t K, int leaf, int* T, int* F, int* L) {
  if (!T || !F || !L) return tbik::set_error(TBIK_ERR_ARG, "tbik_tree_shape: null output pointer");
  int rc = tbik::tree_shape(K, leaf, T, F, L);
  if (rc != TBIK_OK) return tbik::set_error(rc, "tbik_tree_shape: K must be a positive multiple of leaf");
  return TBIK_OK;
}

int tbik_gemm(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
              int dtype, int leaf, int node_dtype, tbik_stream_t stream) {
  return tbik::gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0,
                           static_cast<cudaStream_t>(stream));
}

int tbik_gemm_ex(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 int dtype, int leaf, int node_dtype, int max_ctas, tbik_stream_t stream) {
  return tbik::gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, max_ctas,
                           static_cast<cudaStream_t>(stream));
}

int tbik_gemm_status(uint32_t out[4]) {
  if (!out) return tbik::set_error(TBIK_ERR_ARG, "tbik_gemm_status: null output pointer");
  return tbik::gemm_status(out);
}

}  // extern "C"
