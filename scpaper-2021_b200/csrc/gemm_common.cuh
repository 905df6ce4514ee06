// Pieces shared by the GEMM kernels: tile constants, the argument block, and the fp16
// epilogue step (bias, activation, conversion, swizzled staging line).
#pragma once

#include "common.cuh"

namespace et {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = 32 * EPI_WARPS;
constexpr int GEMM_THREADS = 64 + EPI_THREADS;
constexpr int A_STAGE_BYTES = BM * BK * 2;

enum : int { OUT_TILE_F16 = 0, OUT_INDEXED = 1, OUT_GROUPED = 2, OUT_PARTIAL_F32 = 3 };

// Tiles are numbered t = (z * tiles_m + m) * tiles_n + n.  z selects a group (B_MN: z-th
// weight matrix / bias, output rows interleaved: row m of group z lands at
// (m / grp_rows) * grp_stride + z * grp_rows + m % grp_rows) or a K split (OUT_PARTIAL_F32:
// K blocks [z * kb_per_split, (z + 1) * kb_per_split)).
struct GemmArgs {
    void* Y;
    const __half* bias;
    const int* col_map;
    int ldy, scatter, M, N, K, act;
    int grp_rows, grp_stride;
    int out_mode;
    int kb_per_split;
    int nz;  // groups or splits
    int* err_word;
};

template <int ACT>
__device__ __forceinline__ float act_fn(float x) {
    if (ACT == ET_ACT_RELU) return fmaxf(x, 0.f);
    if (ACT == ET_ACT_GELU) return gelu_tanh(x);
    return x;
}

// 32 accumulator columns of one row -> bias, activation, fp16 -> four swizzled 16-byte
// chunks of the row's 128-byte staging line (half 0 or 1 of a 64-column group).
template <int ACT>
__device__ __forceinline__ void stage_f16_chunk(const uint32_t (&r)[32], const float* bias32,
                                                uint8_t* srow, int half, int lane) {
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
        const float4 b0 = *reinterpret_cast<const float4*>(bias32 + gq * 8);
        const float4 b1 = *reinterpret_cast<const float4*>(bias32 + gq * 8 + 4);
        float v[8];
        v[0] = __uint_as_float(r[gq * 8 + 0]) + b0.x;
        v[1] = __uint_as_float(r[gq * 8 + 1]) + b0.y;
        v[2] = __uint_as_float(r[gq * 8 + 2]) + b0.z;
        v[3] = __uint_as_float(r[gq * 8 + 3]) + b0.w;
        v[4] = __uint_as_float(r[gq * 8 + 4]) + b1.x;
        v[5] = __uint_as_float(r[gq * 8 + 5]) + b1.y;
        v[6] = __uint_as_float(r[gq * 8 + 6]) + b1.z;
        v[7] = __uint_as_float(r[gq * 8 + 7]) + b1.w;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = act_fn<ACT>(v[j]);
        uint4 o;
        o.x = pack_half2(v[0], v[1]);
        o.y = pack_half2(v[2], v[3]);
        o.z = pack_half2(v[4], v[5]);
        o.w = pack_half2(v[6], v[7]);
        const int chunk = ((half << 2) + gq) ^ (lane & 7);
        *reinterpret_cast<uint4*>(srow + chunk * 16) = o;
    }
}


// Tensor map of a K-major operand [rows, K] (leading dimension ld) read in 64 x box_rows boxes.
inline int encode_operand(CUtensorMap* tm, const __half* p, int ld, int rows, int K, int box_rows) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ld) * 2};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(box_rows)};
    return make_tensor_map_f16(tm, p, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace gemm
}  // namespace et
