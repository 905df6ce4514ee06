// culib::cuda_map / cuda_vecadd with the reference's call forms (lib/cuda_map.cuh:11-27):
// data[i] = op(data, i) for i < len with a device lambda (compile with --extended-lambda).
// The operators of this library do not use it (bias, activation and scaling live in their
// kernels' epilogues); it is here for driver code written against the reference.
#pragma once
#include <cuda_runtime.h>

template <typename T, typename F>
__global__ void __kernel__cuda_map(T* data, const int len, F op) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < len; i += blockDim.x * gridDim.x)
        data[i] = op(data, i);
}

namespace culib {

template <typename T, typename F>
void cuda_map(T* data, const int len, F op, cudaStream_t stream = 0) {
    if (len <= 0) return;
    const int threads = 256;
    int blocks = (len + threads - 1) / threads;
    if (blocks > 148 * 8) blocks = 148 * 8;
    __kernel__cuda_map<<<blocks, threads, 0, stream>>>(data, len, op);
}

// A = A + B (a device lambda: available when the translation unit is compiled with
// --extended-lambda, as the reference's build does)
#if defined(__CUDACC_EXTENDED_LAMBDA__)
template <typename T>
void cuda_vecadd(T* A, const T* B, const int size, cudaStream_t stream = 0) {
    const auto add_op = [B] __device__(T * data, int i) -> T { return data[i] + B[i]; };
    cuda_map(A, size, add_op, stream);
}
#endif

}  // namespace culib
