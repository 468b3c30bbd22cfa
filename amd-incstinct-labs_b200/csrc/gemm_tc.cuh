// Interface of the tensor-core GEMM (gemm_tc.cu) for the other translation units of the library.
#pragma once
#include <cuda_runtime.h>

namespace b200p {

// Epilogues: numbered like the skinny GEMM's (b200p_skinny_gemm).
enum GemmEpilogue { GEMM_EPI_STORE16 = 0, GEMM_EPI_ACC32 = 1, GEMM_EPI_STORE32 = 2, GEMM_EPI_SILU16 = 3 };

// C[M,N] = A[M,K] . W[N,K]^T (see b200p_gemm_16).  Status code; nothing is launched on an error.
int gemm_tc(int dtype, int epi, const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
            long long ldc, cudaStream_t st);

} // namespace b200p
