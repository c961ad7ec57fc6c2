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
  return tbik::gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0, 0, nullptr, 0,
                           static_cast<cudaStream_t>(stream), 1);
}

size_t tbik_gemm_workspace_bytes(int M, int N, int64_t K, int leaf) { return tbik::gemm_workspace_bytes(M, N, K, leaf); }

int tbik_gemm_ws(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 int dtype, int leaf, int node_dtype, void* workspace, size_t workspace_bytes, tbik_stream_t stream) {
  return tbik::gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0, 0, workspace, workspace_bytes,
                           static_cast<cudaStream_t>(stream), 0);
}

int tbik_gemm_ex(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 int dtype, int leaf, int node_dtype, int max_ctas, int tiling, void* workspace, size_t workspace_bytes,
                 tbik_stream_t stream) {
  return tbik::gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, max_ctas, tiling, workspace,
                           workspace_bytes, static_cast<cudaStream_t>(stream), tiling == 0 ? 0 : 1);
}

int tbik_gemm_plan(int M, int N, int64_t K, int leaf, int max_ctas, size_t workspace_bytes, int out[4]) {
  if (!out) return tbik::set_error(TBIK_ERR_ARG, "tbik_gemm_plan: null output pointer");
  return tbik::gemm_plan_query(M, N, K, leaf, max_ctas, workspace_bytes, out);
}

size_t tbik_gemm_slabs_workspace_bytes(int M, int N, int64_t K, int leaf, int tiling, int slabs) {
  return tbik::gemm_split_workspace_bytes(M, N, K, leaf, tiling, slabs);
}

int tbik_gemm_slabs(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                    int dtype, int leaf, int node_dtype, int tiling, int slabs, void* workspace, size_t workspace_bytes,
                    tbik_stream_t stream) {
  if (tiling < 1) return tbik::set_error(TBIK_ERR_ARG, "tbik_gemm_slabs: an explicit tiling (1..6) is required");
  if (slabs < 1) return tbik::set_error(TBIK_ERR_ARG, "tbik_gemm_slabs: slabs must be >= 1");
  return tbik::gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0, tiling, workspace,
                           workspace_bytes, static_cast<cudaStream_t>(stream), slabs);
}

size_t tbik_gemm_static_scratch_bytes(void) { return tbik::gemm_static_scratch_bytes(); }

int tbik_gemm_static_accepts(int M, int N, int64_t K, int leaf) { return tbik::gemm_static_accepts(M, N, K, leaf); }

int tbik_gemm_static(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                     int dtype, int leaf, int node_dtype, tbik_stream_t stream) {
  return tbik::gemm_launch_static(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype,
                                  static_cast<cudaStream_t>(stream));
}

int tbik_gemm_status(uint32_t out[4]) {
  if (!out) return tbik::set_error(TBIK_ERR_ARG, "tbik_gemm_status: null output pointer");
  return tbik::gemm_status(out);
}


size_t tbik_ar_meta_size(void) { return tbik::ar_meta_size(); }

int tbik_ar_create(void* const* signals, int world, int rank, void* rank_data, size_t rank_data_bytes,
                   int full_nvlink, tbik_ar_t* out) {
  return tbik::ar_create(signals, world, rank, rank_data, rank_data_bytes, full_nvlink, out);
}

int tbik_ar_destroy(tbik_ar_t comm) { return tbik::ar_destroy(comm); }

int tbik_ar_configure(tbik_ar_t comm, int key, int64_t value) { return tbik::ar_configure(comm, key, value); }

int tbik_ar_register_buffer(tbik_ar_t comm, void* const* ptrs) { return tbik::ar_register_buffer(comm, ptrs); }

int tbik_ar_tree_allreduce(tbik_ar_t comm, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer,
                           size_t reg_buffer_bytes, tbik_stream_t stream) {
  return tbik::ar_run(comm, inp, out, numel, dtype, reg_buffer, reg_buffer_bytes, true,
                      static_cast<cudaStream_t>(stream));
}

int tbik_ar_allreduce(tbik_ar_t comm, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer,
                      size_t reg_buffer_bytes, tbik_stream_t stream) {
  return tbik::ar_run(comm, inp, out, numel, dtype, reg_buffer, reg_buffer_bytes, false,
                      static_cast<cudaStream_t>(stream));
}

int tbik_ar_tree_allreduce_within(tbik_ar_t comm, const void* reg_base, size_t byte_offset, void* out, int64_t numel,
                                  int dtype, tbik_stream_t stream) {
  return tbik::ar_run_within(comm, reg_base, byte_offset, out, numel, dtype, static_cast<cudaStream_t>(stream));
}

int tbik_ar_tree_allreduce_rounding(tbik_ar_t comm, const void* reg_base, size_t byte_offset, void* out, int64_t numel,
                                    int out_dtype, void* stream) {
  return tbik::ar_run_rounding(comm, reg_base, byte_offset, out, numel, out_dtype, static_cast<cudaStream_t>(stream));
}

int tbik_ar_row_split_layer(tbik_ar_t comm, const void* A, const void* W, void* out, int M, int N, int K, int64_t lda,
                            int64_t ldw, int dtype, int leaf, void* reg_base, size_t reg_bytes, void* workspace,
                            size_t workspace_bytes, const int* block_rows, int num_blocks, int comm_ctas,
                            tbik_stream_t main_stream, tbik_stream_t side_stream) {
  return tbik::ar_row_split_layer(comm, A, W, out, M, N, K, lda, ldw, dtype, leaf, reg_base, reg_bytes, workspace,
                                  workspace_bytes, block_rows, num_blocks, comm_ctas, static_cast<cudaStream_t>(main_stream),
                                  static_cast<cudaStream_t>(side_stream));
}

int tbik_ar_trace(tbik_ar_t comm, uint64_t* out, int max_blocks, int* blocks) {
  return tbik::ar_trace(comm, out, max_blocks, blocks);
}

int tbik_ar_graph_meta_count(tbik_ar_t comm, int* n) { return tbik::ar_graph_meta_count(comm, n); }

int tbik_ar_graph_meta(tbik_ar_t comm, void* handles_out, int64_t* offsets_out) {
  return tbik::ar_graph_meta(comm, handles_out, offsets_out);
}

int tbik_ar_register_graph_buffers(tbik_ar_t comm, const void* const* handles, const int64_t* const* offsets) {
  return tbik::ar_register_graph_buffers(comm, handles, offsets);
}

int tbik_ar_status(tbik_ar_t comm, uint32_t out[8]) { return tbik::ar_status(comm, out); }

}  // extern "C"
