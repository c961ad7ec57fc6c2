// Declarations shared by the translation units of libtbik_b200.so (not part of the C ABI).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tbik.h"

namespace tbik {

// Records `msg` as the calling thread's last error and returns `code`.
int set_error(int code, const char* msg);
int set_cuda_error(cudaError_t e, const char* what);

int tree_shape(int64_t K, int leaf, int* T, int* F, int* L);
int gemm_launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                int dtype, int leaf, int node_dtype, int max_ctas, int tiling, void* workspace, size_t ws_bytes,
                cudaStream_t stream, int splits);  // splits: 0 = automatic (tiling 0 only), 1 = none, 2..16 = K-slabs
size_t gemm_workspace_bytes(int M, int N, int64_t K, int leaf);
int gemm_plan_query(int M, int N, int64_t K, int leaf, int max_ctas, size_t ws_bytes, int out[4]);
size_t gemm_split_workspace_bytes(int M, int N, int64_t K, int leaf, int tiling, int splits);
size_t gemm_static_scratch_bytes();
int gemm_static_accepts(int M, int N, int64_t K, int leaf);

int gemm_launch_static(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                       int64_t ldc, int dtype, int leaf, int node_dtype, cudaStream_t stream);
int gemm_status(uint32_t out[4]);


size_t ar_meta_size();
int ar_create(void* const* signals, int world, int rank, void* rank_data, size_t rank_data_bytes, int full_nvlink,
              tbik_ar_t* out);
int ar_destroy(tbik_ar_t h);
int ar_configure(tbik_ar_t h, int key, int64_t value);
int ar_register_buffer(tbik_ar_t h, void* const* ptrs);
int ar_run(tbik_ar_t h, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer, size_t reg_bytes,
           bool tree, cudaStream_t stream);
int ar_run_within(tbik_ar_t h, const void* reg_base, size_t byte_offset, void* out, int64_t numel, int dtype,
                  cudaStream_t stream);
int ar_run_rounding(tbik_ar_t h, const void* reg_base, size_t byte_offset, void* out, int64_t numel, int out_dtype,
                    cudaStream_t stream);
int ar_row_split_layer(tbik_ar_t h, const void* A, const void* W, void* out, int M, int N, int K, int64_t lda,
                       int64_t ldw, int dtype, int leaf, void* reg_base, size_t reg_bytes, void* workspace,
                       size_t ws_bytes, const int* block_rows, int nblk, int comm_ctas, cudaStream_t main,
                       cudaStream_t side);
int ar_trace(tbik_ar_t h, uint64_t* out, int max_blocks, int* blocks);
int ar_graph_meta_count(tbik_ar_t h, int* n);
int ar_graph_meta(tbik_ar_t h, void* handles_out, int64_t* offsets_out);
int ar_register_graph_buffers(tbik_ar_t h, const void* const* handles, const int64_t* const* offsets);
int ar_status(tbik_ar_t h, uint32_t out[8]);

}  // namespace tbik
