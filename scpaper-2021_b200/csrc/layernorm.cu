// Residual-add + LayerNorm, plain LayerNorm, and the stand-alone element-wise passes
// (activation, bias add).  All are HBM-bound: 128-bit loads and stores, fp32 statistics
// reduced with warp shuffles, one warp per token row.
#include "common.cuh"
#include "kernels.h"

namespace et {

namespace {

constexpr int LN_WARPS = 4;
constexpr int LN_MAX_CHUNKS = 8;  // per lane, 8 halves each: rows up to 2048 stay in registers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
    }
}

// size % 8 == 0.  Variance as E[x^2] - E[x]^2 in fp32, clamped at zero.
// NCH: chunks of 8 halves per lane kept in registers (rows up to NCH * 256), 0 = any size,
// the row is read twice.
template <int NCH>
__global__ void __launch_bounds__(LN_WARPS * 32)
skip_layernorm_kernel(const __half* __restrict__ src, const __half* __restrict__ skip,
                      const __half* __restrict__ gamma, const __half* __restrict__ beta,
                      __half* __restrict__ out, int rows, int size, float eps) {
    constexpr bool CACHED = NCH > 0;
    constexpr int LN_CH = CACHED ? NCH : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * LN_WARPS + warp;
    const int nchunk = size >> 3;
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    const uint4* b4 = reinterpret_cast<const uint4*>(beta);
    // gamma / beta are weights: fetch them before waiting for the kernel that produces src,
    // so that their L2 round trip is off the critical path
    uint4 gq[LN_CH], bq[LN_CH];
    if (CACHED) {
#pragma unroll
        for (int it = 0; it < LN_CH; ++it) {
            const int c = lane + it * 32;
            if (c < nchunk) {
                gq[it] = __ldg(g4 + c);
                bq[it] = __ldg(b4 + c);
            }
        }
    }
    pdl_launch_dependents();
    pdl_wait();
    if (row >= rows) return;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + static_cast<size_t>(row) * size);
    const uint4* k4 =
        skip ? reinterpret_cast<const uint4*>(skip + static_cast<size_t>(row) * size) : nullptr;
    uint4* o4 = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * size);

    float cache[LN_CH][8];
    float sum = 0.f, sq = 0.f;
    // CACHED: static trip count so the row stays in registers; otherwise a plain strided loop.
    const int trips = CACHED ? LN_CH : (nchunk + 31) / 32;
#pragma unroll
    for (int it = 0; it < (CACHED ? LN_CH : trips); ++it) {
        const int c = lane + it * 32;
        if (c < nchunk) {
            float v[8];
            unpack8(__ldcg(s4 + c), v);
            if (k4) {
                float w[8];
                unpack8(__ldcg(k4 + c), w);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += w[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sum += v[j];
                sq += v[j] * v[j];
                if (CACHED) cache[it][j] = v[j];
            }
        }
    }
    sum = warp_sum(sum);
    sq = warp_sum(sq);
    const float mean = sum / size;
    const float var = fmaxf(sq / size - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);

#pragma unroll
    for (int it = 0; it < (CACHED ? LN_CH : trips); ++it) {
        const int c = lane + it * 32;
        if (c < nchunk) {
            float v[8];
            if (CACHED) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = cache[it][j];
            } else {
                unpack8(__ldcg(s4 + c), v);
                if (k4) {
                    float w[8];
                    unpack8(__ldcg(k4 + c), w);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] += w[j];
                }
            }
            float g[8], b[8];
            unpack8(CACHED ? gq[it] : __ldg(g4 + c), g);
            unpack8(CACHED ? bq[it] : __ldg(b4 + c), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (v[j] - mean) * rstd * g[j] + b[j];
            uint4 o;
            o.x = pack_half2(v[0], v[1]);
            o.y = pack_half2(v[2], v[3]);
            o.z = pack_half2(v[4], v[5]);
            o.w = pack_half2(v[6], v[7]);
            o4[c] = o;
        }
    }
}

// Same normalisation fed by split-K partial sums: the row is
//   sum_p partials[p][row, :] + bias + skip[row, :]
// so the GEMM that precedes it never rounds its result to fp16 nor adds its bias.
__global__ void __launch_bounds__(LN_WARPS * 32)
skip_layernorm_partials_kernel(const float* __restrict__ partials, int nsplit, size_t split_stride,
                               const __half* __restrict__ bias, const __half* __restrict__ skip,
                               const __half* __restrict__ gamma, const __half* __restrict__ beta,
                               __half* __restrict__ out, int rows, int size, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * LN_WARPS + warp;
    pdl_launch_dependents();
    pdl_wait();
    if (row >= rows) return;
    const int nchunk = size >> 3;
    const uint4* k4 =
        skip ? reinterpret_cast<const uint4*>(skip + static_cast<size_t>(row) * size) : nullptr;
    uint4* o4 = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * size);
    float cache[LN_MAX_CHUNKS][8];
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int it = 0; it < LN_MAX_CHUNKS; ++it) {
        const int c = lane + it * 32;
        if (c < nchunk) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
            for (int p = 0; p < nsplit; ++p) {
                const float4* src = reinterpret_cast<const float4*>(
                    partials + p * split_stride + static_cast<size_t>(row) * size + c * 8);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
            }
            float w[8];
            if (bias) {
                unpack8(__ldg(reinterpret_cast<const uint4*>(bias) + c), w);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += w[j];
            }
            if (k4) {
                unpack8(__ldcg(k4 + c), w);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += w[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sum += v[j];
                sq += v[j] * v[j];
                cache[it][j] = v[j];
            }
        }
    }
    sum = warp_sum(sum);
    sq = warp_sum(sq);
    const float mean = sum / size;
    const float var = fmaxf(sq / size - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);
#pragma unroll
    for (int it = 0; it < LN_MAX_CHUNKS; ++it) {
        const int c = lane + it * 32;
        if (c < nchunk) {
            float g[8], b[8], v[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + c), g);
            unpack8(__ldg(reinterpret_cast<const uint4*>(beta) + c), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (cache[it][j] - mean) * rstd * g[j] + b[j];
            uint4 o;
            o.x = pack_half2(v[0], v[1]);
            o.y = pack_half2(v[2], v[3]);
            o.z = pack_half2(v[4], v[5]);
            o.w = pack_half2(v[6], v[7]);
            o4[c] = o;
        }
    }
}

// in and out may be the same buffer (the reference applies the activation in place).
__global__ void act_kernel(const __half* in, __half* out, size_t n, int act) {
    const size_t n8 = n >> 3;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
         i += stride) {
        float v[8];
        unpack8(reinterpret_cast<const uint4*>(in)[i], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = apply_act(v[j], act);
        uint4 o;
        o.x = pack_half2(v[0], v[1]);
        o.y = pack_half2(v[2], v[3]);
        o.z = pack_half2(v[4], v[5]);
        o.w = pack_half2(v[6], v[7]);
        reinterpret_cast<uint4*>(out)[i] = o;
    }
    // ragged tail (n % 8 values)
    for (size_t i = (n8 << 3) + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += stride)
        out[i] = __float2half_rn(apply_act(__half2float(in[i]), act));
}

__global__ void bias_add_kernel(__half* __restrict__ data, const __half* __restrict__ bias,
                                int rows, int cols) {
    const size_t n8 = static_cast<size_t>(rows) * cols / 8;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>((i * 8) % cols);
        float v[8], b[8];
        unpack8(reinterpret_cast<const uint4*>(data)[i], v);
        unpack8(__ldg(reinterpret_cast<const uint4*>(bias + c)), b);
        uint4 o;
        o.x = pack_half2(v[0] + b[0], v[1] + b[1]);
        o.y = pack_half2(v[2] + b[2], v[3] + b[3]);
        o.z = pack_half2(v[4] + b[4], v[5] + b[5]);
        o.w = pack_half2(v[6] + b[6], v[7] + b[7]);
        reinterpret_cast<uint4*>(data)[i] = o;
    }
}

int grid_for(size_t work_items, int threads, int cap) {
    size_t b = (work_items + threads - 1) / threads;
    if (b < 1) b = 1;
    return static_cast<int>(b < static_cast<size_t>(cap) ? b : cap);
}

}  // namespace

int launch_skip_layernorm(const __half* src, const __half* skip, const __half* gamma,
                          const __half* beta, __half* out, int rows, int size,
                          cudaStream_t stream) {
    if (!src || !gamma || !beta || !out || rows <= 0 || size <= 0) return ET_ERR_INVALID_ARG;
    if (size % 8) return ET_ERR_SHAPE;
    if (!aligned16(src) || !aligned16(out) || !aligned16(gamma) || !aligned16(beta) ||
        (skip && !aligned16(skip)))
        return ET_ERR_ALIGNMENT;
    const int blocks = (rows + LN_WARPS - 1) / LN_WARPS;
    cudaError_t e;
    auto go = [&](auto kern) {
        return launch_kernel(kern, dim3(blocks), dim3(LN_WARPS * 32), 0, stream, src, skip, gamma,
                             beta, out, rows, size, 1e-5f);
    };
    if (size <= 3 * 256)
        e = go(skip_layernorm_kernel<3>);
    else if (size <= 4 * 256)
        e = go(skip_layernorm_kernel<4>);
    else if (size <= LN_MAX_CHUNKS * 256)
        e = go(skip_layernorm_kernel<LN_MAX_CHUNKS>);
    else
        e = go(skip_layernorm_kernel<0>);
    return e == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int launch_skip_layernorm_partials(const float* partials, int nsplit, size_t split_stride,
                                   const __half* bias, const __half* skip, const __half* gamma,
                                   const __half* beta, __half* out, int rows, int size,
                                   cudaStream_t stream) {
    if (!partials || !gamma || !beta || !out || rows <= 0 || size <= 0 || nsplit <= 0)
        return ET_ERR_INVALID_ARG;
    if (size % 8 || size > LN_MAX_CHUNKS * 8 * 32) return ET_ERR_SHAPE;
    const int blocks = (rows + LN_WARPS - 1) / LN_WARPS;
    return launch_kernel(skip_layernorm_partials_kernel, dim3(blocks), dim3(LN_WARPS * 32), 0,
                         stream, partials, nsplit, split_stride, bias, skip, gamma, beta, out, rows,
                         size, 1e-5f) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

}  // namespace et

extern "C" {

int et_skip_layernorm_fwd(const et_half* src, const et_half* skip, const et_half* gamma,
                          const et_half* beta, et_half* out, int rows, int size,
                          et_stream stream) {
    if (!skip) return ET_ERR_INVALID_ARG;
    return et::launch_skip_layernorm(
        reinterpret_cast<const __half*>(src), reinterpret_cast<const __half*>(skip),
        reinterpret_cast<const __half*>(gamma), reinterpret_cast<const __half*>(beta),
        reinterpret_cast<__half*>(out), rows, size, static_cast<cudaStream_t>(stream));
}

int et_layernorm_fwd(const et_half* src, const et_half* gamma, const et_half* beta, et_half* out,
                     int rows, int size, et_stream stream) {
    return et::launch_skip_layernorm(reinterpret_cast<const __half*>(src), nullptr,
                                     reinterpret_cast<const __half*>(gamma),
                                     reinterpret_cast<const __half*>(beta),
                                     reinterpret_cast<__half*>(out), rows, size,
                                     static_cast<cudaStream_t>(stream));
}

int et_act_fwd(const et_half* in, et_half* out, size_t n, int act, et_stream stream) {
    if (!in || !out || n == 0) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (!et::aligned16(in) || !et::aligned16(out)) return ET_ERR_ALIGNMENT;
    et::count_launch();
    et::act_kernel<<<et::grid_for(n / 8 + 1, 256, 148 * 8), 256, 0,
                     static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const __half*>(in),
                                                          reinterpret_cast<__half*>(out), n, act);
    return cudaGetLastError() == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

int et_bias_add_fwd(et_half* data, const et_half* bias, int rows, int cols, et_stream stream) {
    if (!data || !bias || rows <= 0 || cols <= 0) return ET_ERR_INVALID_ARG;
    if (cols % 8) return ET_ERR_SHAPE;
    if (!et::aligned16(data) || !et::aligned16(bias)) return ET_ERR_ALIGNMENT;
    et::count_launch();
    et::bias_add_kernel<<<et::grid_for(static_cast<size_t>(rows) * cols / 8, 256, 148 * 8), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<__half*>(data), reinterpret_cast<const __half*>(bias), rows, cols);
    return cudaGetLastError() == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

}  // extern "C"
