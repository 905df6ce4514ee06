// Linear layers over the irregular weight formats, on CUDA cores:
//   - 1x16 vectors (mat1x16): one thread per token accumulates the 16 outputs of a row
//     set, walking the stored vectors of each 16-column part;
//   - CSR: a CTA keeps 8 token rows in shared memory and its threads sweep the output
//     features, gathering activations by column index.
// Irregular sparsity has no dense sub-blocks to hand to the tensor cores; these kernels
// exist so every reference format computes the right result.
#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

constexpr int V16_THREADS = 128;

__global__ void __launch_bounds__(V16_THREADS)
linear_1x16_kernel(const int* __restrict__ tile_idx, const int* __restrict__ row_idx,
                   const __half* __restrict__ data, const __half* __restrict__ bias,
                   const __half* __restrict__ X, __half* __restrict__ Y, int T, int in, int out,
                   int act) {
    const int rset = blockIdx.x;
    const int t = blockIdx.y * V16_THREADS + threadIdx.x;
    const int npart = in >> 4;
    const int* tidx = tile_idx + static_cast<size_t>(rset) * (npart + 1);
    float acc[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) acc[q] = 0.f;
    const bool live = t < T;
    const __half* xrow = X + static_cast<size_t>(live ? t : 0) * in;
    for (int p = 0; p < npart; ++p) {
        const int beg = __ldg(tidx + p), end = __ldg(tidx + p + 1);
        if (beg >= end) continue;  // uniform over the CTA
        float x[16];
        {
            const uint4 a = __ldcg(reinterpret_cast<const uint4*>(xrow + p * 16));
            const uint4 b = __ldcg(reinterpret_cast<const uint4*>(xrow + p * 16 + 8));
            const __half2* ha = reinterpret_cast<const __half2*>(&a);
            const __half2* hb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
                x[2 * j] = fa.x;
                x[2 * j + 1] = fa.y;
                x[8 + 2 * j] = fb.x;
                x[8 + 2 * j + 1] = fb.y;
            }
        }
        for (int i = beg; i < end; ++i) {
            const int q = __ldg(row_idx + i) & 15;
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(data + static_cast<size_t>(i) * 16));
            const uint4 b =
                __ldg(reinterpret_cast<const uint4*>(data + static_cast<size_t>(i) * 16 + 8));
            const __half2* ha = reinterpret_cast<const __half2*>(&a);
            const __half2* hb = reinterpret_cast<const __half2*>(&b);
            float dot = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
                dot += fa.x * x[2 * j] + fa.y * x[2 * j + 1];
                dot += fb.x * x[8 + 2 * j] + fb.y * x[8 + 2 * j + 1];
            }
#pragma unroll
            for (int qq = 0; qq < 16; ++qq) acc[qq] += (q == qq) ? dot : 0.f;
        }
    }
    if (!live) return;
    float f[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) {
        const float b = bias ? __half2float(__ldg(bias + rset * 16 + q)) : 0.f;
        f[q] = apply_act(acc[q] + b, act);
    }
    uint4 o0, o1;
    o0.x = pack_half2(f[0], f[1]);
    o0.y = pack_half2(f[2], f[3]);
    o0.z = pack_half2(f[4], f[5]);
    o0.w = pack_half2(f[6], f[7]);
    o1.x = pack_half2(f[8], f[9]);
    o1.y = pack_half2(f[10], f[11]);
    o1.z = pack_half2(f[12], f[13]);
    o1.w = pack_half2(f[14], f[15]);
    __half* y = Y + static_cast<size_t>(t) * out + rset * 16;
    *reinterpret_cast<uint4*>(y) = o0;
    *reinterpret_cast<uint4*>(y + 8) = o1;
}

constexpr int CSR_TOKENS = 8;
constexpr int CSR_THREADS = 256;

__global__ void __launch_bounds__(CSR_THREADS)
linear_csr_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const __half* __restrict__ data, const __half* __restrict__ bias,
                  const __half* __restrict__ X, __half* __restrict__ Y, int T, int in, int out,
                  int act) {
    extern __shared__ __half xs[];  // [CSR_TOKENS][in]
    const int t0 = blockIdx.x * CSR_TOKENS;
    const int nt = (T - t0) < CSR_TOKENS ? (T - t0) : CSR_TOKENS;
    const int chunks = in >> 3;
    for (int i = threadIdx.x; i < CSR_TOKENS * chunks; i += CSR_THREADS) {
        const int tt = i / chunks, c = i - tt * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tt < nt) v = __ldcg(reinterpret_cast<const uint4*>(X + static_cast<size_t>(t0 + tt) * in) + c);
        reinterpret_cast<uint4*>(xs + static_cast<size_t>(tt) * in)[c] = v;
    }
    __syncthreads();
    for (int o = threadIdx.x; o < out; o += CSR_THREADS) {
        float acc[CSR_TOKENS];
#pragma unroll
        for (int tt = 0; tt < CSR_TOKENS; ++tt) acc[tt] = 0.f;
        const int beg = __ldg(indptr + o), end = __ldg(indptr + o + 1);
        for (int i = beg; i < end; ++i) {
            const float w = __half2float(__ldg(data + i));
            const int c = __ldg(indices + i);
#pragma unroll
            for (int tt = 0; tt < CSR_TOKENS; ++tt)
                acc[tt] += w * __half2float(xs[static_cast<size_t>(tt) * in + c]);
        }
        const float b = bias ? __half2float(__ldg(bias + o)) : 0.f;
#pragma unroll
        for (int tt = 0; tt < CSR_TOKENS; ++tt)
            if (tt < nt)
                Y[static_cast<size_t>(t0 + tt) * out + o] = __float2half_rn(apply_act(acc[tt] + b, act));
    }
}

// One CTA per 16-row set: dense[set * 16 + q][part * 16 .. + 16] = data[i] for every stored
// vector i of the set (q = row_idx[i] % 16); thread = (vector slot in a group of 16, element).
__global__ void densify_1x16_kernel(const int* __restrict__ tile_idx, const int* __restrict__ row_idx,
                                    const __half* __restrict__ data, int npart, int in,
                                    __half* __restrict__ dense) {
    const int rset = blockIdx.x;
    const int* tidx = tile_idx + static_cast<size_t>(rset) * (npart + 1);
    const int beg0 = __ldg(tidx), end0 = __ldg(tidx + npart);
    const int j = threadIdx.x & 15;
    for (int i = beg0 + (threadIdx.x >> 4); i < end0; i += blockDim.x >> 4) {
        // the part of vector i: the last p with tile_idx[p] <= i (binary search)
        int lo = 0, hi = npart - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(tidx + mid) <= i) lo = mid; else hi = mid - 1;
        }
        const int q = __ldg(row_idx + i) & 15;
        dense[(static_cast<size_t>(rset) * 16 + q) * in + lo * 16 + j] = data[static_cast<size_t>(i) * 16 + j];
    }
}

}  // namespace
}  // namespace et

extern "C" {

int et_1x16_prefer_dense(int in, int out, int nvec) {
    if (in <= 0 || out <= 0 || (in & 15) || (out & 15)) return 0;
    // a stored vector costs the CUDA-core kernel 16 multiply-adds per token, a dense 16 x 16
    // tile costs the tensor core a sixteenth of a cycle per token: dense wins unless almost
    // nothing is stored
    const double total = static_cast<double>(out) * (in >> 4);
    return nvec > 0.01 * total ? 1 : 0;
}

int et_1x16_densify(const int32_t* tile_idx, const int32_t* row_idx, const et_half* data, int nvec,
                    int in, int out, et_half* dense, et_stream stream) {
    if (!tile_idx || !dense || in <= 0 || out <= 0 || nvec < 0) return ET_ERR_INVALID_ARG;
    if ((in & 15) || (out & 15)) return ET_ERR_SHAPE;
    if (nvec > 0 && (!row_idx || !data)) return ET_ERR_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(dense, 0, static_cast<size_t>(in) * out * sizeof(__half), s) != cudaSuccess)
        return ET_ERR_CUDA;
    if (nvec > 0) {
        et::count_launch();
        et::densify_1x16_kernel<<<out >> 4, 256, 0, s>>>(tile_idx, row_idx,
                                                          reinterpret_cast<const __half*>(data),
                                                          in >> 4, in, reinterpret_cast<__half*>(dense));
        if (cudaGetLastError() != cudaSuccess) return ET_ERR_CUDA;
    }
    return ET_OK;
}

int et_linear_1x16_fwd(const int32_t* tile_idx, const int32_t* row_idx, const et_half* data,
                       int nvec, const et_half* bias, const et_half* X, et_half* Y, int T, int in,
                       int out, int act, et_stream stream) {
    if (!tile_idx || !X || !Y || T <= 0 || in <= 0 || out <= 0 || nvec < 0)
        return ET_ERR_INVALID_ARG;
    if (nvec > 0 && (!row_idx || !data)) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16) return ET_ERR_SHAPE;
    if (!et::aligned16(X) || !et::aligned16(Y) || (data && !et::aligned16(data)))
        return ET_ERR_ALIGNMENT;
    dim3 grid(out / 16, (T + et::V16_THREADS - 1) / et::V16_THREADS);
    if (grid.y > 65535) return ET_ERR_SHAPE;
    et::count_launch();
    et::linear_1x16_kernel<<<grid, et::V16_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        tile_idx, row_idx, reinterpret_cast<const __half*>(data),
        reinterpret_cast<const __half*>(bias), reinterpret_cast<const __half*>(X),
        reinterpret_cast<__half*>(Y), T, in, out, act);
    return cudaGetLastError() == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int et_linear_csr_fwd(const int32_t* indptr, const int32_t* indices, const et_half* data,
                      int nnz, const et_half* bias, const et_half* X, et_half* Y, int T, int in,
                      int out, int act, et_stream stream) {
    if (!indptr || !X || !Y || T <= 0 || in <= 0 || out <= 0 || nnz < 0) return ET_ERR_INVALID_ARG;
    if (nnz > 0 && (!indices || !data)) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (in % 8 || in > 8192) return ET_ERR_SHAPE;
    if (!et::aligned16(X)) return ET_ERR_ALIGNMENT;
    const int smem = et::CSR_TOKENS * in * 2;
    static std::atomic<int> attr_bytes[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && attr_bytes[dev] < smem) {
        if (cudaFuncSetAttribute(et::linear_csr_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem) != cudaSuccess)
            return ET_ERR_CUDA;
        attr_bytes[dev] = smem;
    }
    const int blocks = (T + et::CSR_TOKENS - 1) / et::CSR_TOKENS;
    et::count_launch();
    et::linear_csr_kernel<<<blocks, et::CSR_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(
        indptr, indices, reinterpret_cast<const __half*>(data),
        reinterpret_cast<const __half*>(bias), reinterpret_cast<const __half*>(X),
        reinterpret_cast<__half*>(Y), T, in, out, act);
    return cudaGetLastError() == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

}  // extern "C"
