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
                int dtype, int leaf, int node_dtype, int max_ctas, cudaStream_t stream);
int gemm_status(uint32_t out[4]);

}  // namespace tbik
