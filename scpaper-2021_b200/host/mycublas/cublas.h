// cuBLAS_mmul with the reference's signature (mycublas/cublas.h, mycublas/cublas.cu:4-22):
// row-major C[M, N] = op(A) . op(B), fp16.  The reference forwards to cublasGemmEx; here the
// form every operator of the path uses - A[M, K] times B[N, K] transposed, i.e. a Linear layer
// without bias - runs on this library's own tensor-core GEMM and the handle and algorithm
// arguments are ignored.  Other operand orientations are not part of the hot path and report
// CUBLAS_STATUS_NOT_SUPPORTED.  Only cuBLAS's type definitions are used: nothing here calls
// into or links against cuBLAS.
#pragma once
#include <cublas_v2.h>
#include <cuda_fp16.h>

#include "../lib/utils.h"

inline cublasStatus_t cuBLAS_mmul(const cublasHandle_t& handle, const half* A, const half* B,
                                  half* C, const int M, const int N, const int K,
                                  const bool trans_A, const bool trans_B,
                                  cublasGemmAlgo_t = CUBLAS_GEMM_DEFAULT) {
    if (trans_A || !trans_B) return CUBLAS_STATUS_NOT_SUPPORTED;
    cudaStream_t stream = 0;
    (void)handle;
    const int st = et_linear_dense_fwd(et_ptr(A), et_ptr(B), nullptr, et_ptr(C), M, K, N,
                                       ET_ACT_NONE, stream);
    return st == ET_OK ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_EXECUTION_FAILED;
}
