// Tile-pruned Linear (16x16 tile-CSR, block rows = output features) on tcgen05.
//
// One CTA owns 128 tokens and a panel of 8 output block rows (128 output features,
// 8 x 16 fp32 accumulator columns in tensor memory).  The input is walked in chunks of
// 64 features (4 block columns).  In the prologue the CTA builds, in shared memory, a
// table tile_at[row][block column] of the panel's stored tiles and one 32-bit presence
// mask per chunk (bit = row * 4 + column inside the chunk).  Chunks without any stored
// tile are skipped by every role, so only non-zero tiles and the activations they need are
// loaded.  For a chunk, warp 0 fetches the 128x64 activation slab (TMA, 128-byte swizzle)
// and each stored tile (TMA, 32-byte swizzle: a 16x16 fp16 tile is 16 rows of 32 bytes) into
// densely packed 512-byte slots (16 per stage when no chunk of the panel holds more, else
// 32; the ring gets as many stages as fit); one thread of warp 1 issues one tcgen05.mma
// (M=128, N=16, K=16) per stored tile, choosing the activation slab by descriptor address
// and the accumulator columns by block row; warps 2-9 run the bias / activation / fp16
// epilogue through a swizzled staging tile and TMA stores, writing bias alone for block
// rows that hold no tile.
#include "common.cuh"
#include "kernels.h"

namespace et {

namespace {

// Optional per-CTA timestamps for bring-up builds (-DET_TIMELINE); compiled out otherwise.
#ifdef ET_TIMELINE
__device__ long long et_tile_timeline[4096];
#define ET_TL(slot) \
    if (blockIdx.x == 0 && blockIdx.y == 0) et_tile_timeline[(slot)] = clock64()
#else
#define ET_TL(slot) ((void)0)
#endif

constexpr int TBM = 128;          // tokens per CTA
constexpr int PANEL_ROWS = 8;     // output block rows per CTA
constexpr int TBN = PANEL_ROWS * 16;
constexpr int CHUNK = 64;         // input features per pipeline stage
constexpr int T_EPI_WARPS = 8;
constexpr int T_EPI_THREADS = 32 * T_EPI_WARPS;
constexpr int TILE_THREADS = 64 + T_EPI_THREADS;
constexpr int X_STAGE_BYTES = TBM * CHUNK * 2;  // 16 KB
constexpr int RING_BYTES = 96 * 1024;           // two CTAs per SM
constexpr int MAX_STAGES = 4;
constexpr int MAX_IN = 8192;

__global__ void __launch_bounds__(TILE_THREADS, 2)
linear_tile_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CUtensorMap tmY, const int* __restrict__ row_ptr,
                   const int* __restrict__ row_off, const __half* __restrict__ bias, int T, int in,
                   int out, int act, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int nbc = in >> 4;  // input block columns
    const int nchunk = (in + CHUNK - 1) / CHUNK;
    uint8_t* ring = smem;
    uint8_t* misc = smem + RING_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
    uint64_t* empty_bar = full_bar + MAX_STAGES;
    uint64_t* acc_bar = empty_bar + MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* max_cnt = reinterpret_cast<int*>(tmem_slot + 2);
    int* rp = reinterpret_cast<int*>(tmem_slot + 4);                  // [PANEL_ROWS + 1]
    float* s_bias = reinterpret_cast<float*>(misc + 256);             // [TBN]
    uint32_t* chunk_mask = reinterpret_cast<uint32_t*>(s_bias + TBN);  // [nchunk]
    int* tile_at = reinterpret_cast<int*>(chunk_mask + ((nchunk + 3) & ~3));  // [8][nbc]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int panel = blockIdx.x;
    const int m0 = blockIdx.y * TBM;
    const int n0 = panel * TBN;
    const int nbr = out >> 4;

    // ---- prologue: panel index tables and bias (weights: independent of earlier kernels) ----
    if (threadIdx.x == 0) ET_TL(0);
    if (threadIdx.x <= PANEL_ROWS) {
        int br = panel * PANEL_ROWS + threadIdx.x;
        br = br < nbr ? br : nbr;
        rp[threadIdx.x] = __ldg(row_ptr + br);
    }
    for (int i = threadIdx.x; i < nchunk; i += TILE_THREADS) chunk_mask[i] = 0u;
    for (int i = threadIdx.x; i < TBN; i += TILE_THREADS)
        s_bias[i] = (bias != nullptr && n0 + i < out) ? __half2float(__ldg(bias + n0 + i)) : 0.f;
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmW);
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        *max_cnt = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TBN);
        tmem_relinquish();
    }
    __syncthreads();
    for (int i = rp[0] + threadIdx.x; i < rp[PANEL_ROWS]; i += TILE_THREADS) {
        int r = 0;
        while (r < PANEL_ROWS - 1 && i >= rp[r + 1]) ++r;
        const int off = __ldg(row_off + i);
        if (off >= 0 && off < nbc) {
            tile_at[r * nbc + off] = i;
            atomicOr(&chunk_mask[off >> 2], 1u << (r * 4 + (off & 3)));
        }
    }
    __syncthreads();
    {
        int mc = 0;
        for (int i = threadIdx.x; i < nchunk; i += TILE_THREADS) {
            const int c = __popc(chunk_mask[i]);
            mc = c > mc ? c : mc;
        }
        if (mc > 0) atomicMax(max_cnt, mc);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int panel_tiles = rp[PANEL_ROWS] - rp[0];
    // stage geometry: activation slab + densely packed tile slots
    const int nslot = *max_cnt <= 16 ? 16 : 32;
    const int stage_bytes = X_STAGE_BYTES + nslot * 512;
    const int nstages = RING_BYTES / stage_bytes;  // 4 or 3
    if (threadIdx.x == 0) ET_TL(1);
    pdl_launch_dependents();
    pdl_wait();  // the tables above are weights; activations and Y need the wait

    if (warp == 0) {
        // ---------------- producer (whole warp: lane = row * 4 + column in chunk) ----------------
        const int r = lane >> 2, kb = lane & 3;
        int stage_it = 0;
        bool ok = true;
        for (int kc = 0; kc < nchunk && ok; ++kc) {
            const uint32_t mask = chunk_mask[kc];
            if (mask == 0u) continue;
            const int s = stage_it % nstages;
            const uint32_t ph = (stage_it / nstages) & 1;
            uint8_t* stage = ring + s * stage_bytes;
            if (lane == 0) {
                ok = mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag);
                if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_PRODUCER);
                else
                    mbar_arrive_expect_tx(&full_bar[s], X_STAGE_BYTES + 512u * __popc(mask));
                if (stage_it < 12) ET_TL(16 + stage_it * 4);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) tma_load_2d(stage, &tmX, &full_bar[s], kc * CHUNK, m0);
            if (mask & (1u << lane)) {
                const int t = tile_at[r * nbc + kc * 4 + kb];
                const int slot = __popc(mask & ((1u << lane) - 1u));
                tma_load_2d(stage + X_STAGE_BYTES + slot * 512, &tmW, &full_bar[s], 0, t * 16);
            }
            __syncwarp();
            if (lane == 0 && stage_it < 12) ET_TL(17 + stage_it * 4);
            ++stage_it;
        }
        if (*abort_flag && lane == 0) {
            const int first = stage_it > nstages ? stage_it - nstages : 0;
            for (int it2 = first; it2 < stage_it; ++it2)
                for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                    if (mbar_try_wait(&full_bar[it2 % nstages], (it2 / nstages) & 1)) break;
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (panel_tiles > 0 && elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(TBM, 16, 0, 0);
            uint32_t started = 0;  // bit r: block row r already has a partial sum
            int stage_it = 0;
            bool ok = true;
            for (int kc = 0; kc < nchunk; ++kc) {
                uint32_t mask = chunk_mask[kc];
                if (mask == 0u) continue;
                const int s = stage_it % nstages;
                const uint32_t ph = (stage_it / nstages) & 1;
                if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if (stage_it < 12) ET_TL(18 + stage_it * 4);
                const uint32_t x_addr = smem_u32(ring + s * stage_bytes);
                uint32_t w_addr = x_addr + X_STAGE_BYTES;
                while (mask) {
                    const int bit = __ffs(mask) - 1;
                    mask &= mask - 1;
                    const int r = bit >> 2, kb = bit & 3;
                    const uint64_t ad = make_smem_desc(x_addr + kb * 32, 16, 1024, SWZ_128B);
                    const uint64_t bd = make_smem_desc(w_addr, 16, 256, SWZ_32B);
                    mma_f16_ss(tmem_base + r * 16, ad, bd, idesc, (started >> r) & 1u);
                    started |= 1u << r;
                    w_addr += 512;
                }
                mma_commit(&empty_bar[s]);
                if (stage_it < 12) ET_TL(19 + stage_it * 4);
                ++stage_it;
            }
            if (ok) mma_commit(acc_bar);
            ET_TL(2);
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> staging -> global ----------------
        const int q = warp & 3;            // TMEM lane quadrant
        const int half = (warp - 2) >> 2;  // which 64 output columns of the panel
        bool ok = true;
        if (panel_tiles > 0) {
            ok = mbar_wait_bounded(acc_bar, 0, abort_flag);
            if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_EPILOGUE);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (threadIdx.x == 64) ET_TL(3);
        if (ok && n0 + half * 64 < out) {
            tc_fence_after_sync();
            // every MMA has completed: the ring is idle and serves as the staging area
            uint8_t* tile = ring + (q * 2 + half) * 4096;
            uint8_t* srow = tile + lane * 128;
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = half * 2 + cc;  // 32-column chunk = block rows 2c, 2c + 1
                uint32_t v[32];
                if (panel_tiles > 0) {
                    tmem_ld32(lane_addr + c * 32, v);
                    tmem_ld_wait_regs(v);
                }
                // block rows without a stored tile were never written by the tensor core
                const bool has0 = rp[2 * c + 1] > rp[2 * c], has1 = rp[2 * c + 2] > rp[2 * c + 1];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (!has0) v[j] = 0u;
                    if (!has1) v[16 + j] = 0u;
                }
#pragma unroll
                for (int gq = 0; gq < 4; ++gq) {
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        f[j] = apply_act(__uint_as_float(v[gq * 8 + j]) + s_bias[c * 32 + gq * 8 + j], act);
                    uint4 o;
                    o.x = pack_half2(f[0], f[1]);
                    o.y = pack_half2(f[2], f[3]);
                    o.z = pack_half2(f[4], f[5]);
                    o.w = pack_half2(f[6], f[7]);
                    *reinterpret_cast<uint4*>(srow + ((((cc << 2) + gq) ^ (lane & 7)) * 16)) = o;
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && m0 + q * 32 < T) {
                tma_store_2d(&tmY, tile, n0 + half * 64, m0 + q * 32);
                tma_store_commit();
                tma_store_wait_read();
            }
        }
        if (threadIdx.x == 64) ET_TL(4);
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) ET_TL(5);
    if (warp == 1) tmem_dealloc(tmem_base, TBN);
}

__global__ void tile_fill_bias_kernel(__half* __restrict__ Y, const __half* __restrict__ bias,
                                      size_t rows, int cols, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = rows * cols;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float b = bias ? __half2float(__ldg(bias + (i % cols))) : 0.f;
        Y[i] = __float2half_rn(apply_act(b, act));
    }
}

}  // namespace

int launch_linear_tile(const int* row_ptr, const int* row_off, const __half* tiles, int nnz_tiles,
                       const __half* bias, const __half* X, __half* Y, int T, int in, int out,
                       int act, cudaStream_t stream) {
    if (!row_ptr || !X || !Y || T <= 0 || in <= 0 || out <= 0 || nnz_tiles < 0)
        return ET_ERR_INVALID_ARG;
    if (nnz_tiles > 0 && (!row_off || !tiles)) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16 || in > MAX_IN) return ET_ERR_SHAPE;
    if (!aligned16(X) || !aligned16(Y) || (tiles && !aligned16(tiles)) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;

    if (nnz_tiles == 0) {
        const size_t total = static_cast<size_t>(T) * out;
        const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        return launch_kernel(tile_fill_bias_kernel, dim3(blocks), dim3(256), 0, stream, Y, bias,
                             static_cast<size_t>(T), out, act) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    }

    CUtensorMap tmX, tmW, tmY;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(in), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(in) * 2};
        const uint32_t box[2] = {CHUNK, TBM};
        int st = make_tensor_map_f16(&tmX, X, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    {
        // the tile array seen as a [nnz * 16, 16] matrix: one box = one stored tile
        const uint64_t dims[2] = {16, static_cast<uint64_t>(nnz_tiles) * 16};
        const uint64_t strides[1] = {32};
        const uint32_t box[2] = {16, 16};
        int st = make_tensor_map_f16(&tmW, tiles, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B);
        if (st != ET_OK) return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(out), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(out) * 2};
        const uint32_t box[2] = {64, 32};
        int st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    const int nbc = in / 16, nchunk = (in + CHUNK - 1) / CHUNK;
    const int smem_bytes = RING_BYTES + 256 + TBN * 4 + ((nchunk + 3) & ~3) * 4 +
                           PANEL_ROWS * nbc * 4 + 1024;
    static int attr_bytes[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && attr_bytes[dev] < smem_bytes) {
        if (cudaFuncSetAttribute(linear_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes) != cudaSuccess)
            return ET_ERR_CUDA;
        attr_bytes[dev] = smem_bytes;
    }
    dim3 grid((out + TBN - 1) / TBN, (T + TBM - 1) / TBM);
    return launch_kernel(linear_tile_kernel, grid, dim3(TILE_THREADS), smem_bytes, stream, tmX, tmW,
                         tmY, row_ptr, row_off, bias, T, in, out, act, err) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

}  // namespace et

extern "C" {

int et_linear_tile_fwd(const int32_t* row_ptr, const int32_t* row_off, const et_half* tiles,
                       int nnz_tiles, const et_half* bias, const et_half* X, et_half* Y, int T,
                       int in, int out, int act, et_stream stream) {
    return et::launch_linear_tile(row_ptr, row_off, reinterpret_cast<const __half*>(tiles),
                                  nnz_tiles, reinterpret_cast<const __half*>(bias),
                                  reinterpret_cast<const __half*>(X), reinterpret_cast<__half*>(Y),
                                  T, in, out, act, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
