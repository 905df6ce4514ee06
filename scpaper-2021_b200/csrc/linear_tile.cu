// Tile-pruned Linear (16x16 tile-CSR, block rows = output features) on tcgen05.
//
// One CTA owns 128 tokens and a panel of 8 output block rows (128 output features,
// 8 x 16 fp32 accumulator columns in tensor memory).  The input is walked in chunks of
// 64 features (4 block columns).  In the prologue the CTA builds, in shared memory, a
// table tile_at[row][block column] of the panel's stored tiles and one 32-bit presence
// mask per chunk (bit = row * 4 + column inside the chunk).  Chunks without any stored
// tile are skipped by every role, so only non-zero tiles and the activations they need are
// loaded.  For a chunk, warp 0 fetches the 128x64 activation slab (TMA, 128-byte swizzle)
// and each stored tile (TMA, 32-byte swizzle: a 16x16 fp16 tile is 16 rows of 32 bytes)
// into a per-(row, column) slot; one thread of warp 1 issues one tcgen05.mma
// (M=128, N=16, K=16) per stored tile, choosing the activation slab by descriptor address
// and the accumulator columns by block row; warps 2-5 run the usual bias / activation /
// fp16 epilogue, writing bias alone for block rows that hold no tile.
#include "common.cuh"
#include "kernels.h"

namespace et {

namespace {

constexpr int TBM = 128;          // tokens per CTA
constexpr int PANEL_ROWS = 8;     // output block rows per CTA
constexpr int TBN = PANEL_ROWS * 16;
constexpr int CHUNK = 64;         // input features per pipeline stage
constexpr int TILE_THREADS = 192;
constexpr int X_STAGE_BYTES = TBM * CHUNK * 2;      // 16 KB
constexpr int W_STAGE_BYTES = 32 * 512;             // 32 tile slots of 512 B
constexpr int T_STAGE_BYTES = X_STAGE_BYTES + W_STAGE_BYTES;
constexpr int T_STAGES = 3;
constexpr int MAX_IN = 8192;

__global__ void __launch_bounds__(TILE_THREADS, 2)
linear_tile_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const int* __restrict__ row_ptr, const int* __restrict__ row_off,
                   const __half* __restrict__ bias, __half* __restrict__ Y, int T, int in, int out,
                   int act, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int nbc = in >> 4;                        // input block columns
    const int nchunk = (in + CHUNK - 1) / CHUNK;
    uint8_t* sX = smem;
    uint8_t* sW = smem + T_STAGES * X_STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + T_STAGES * T_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + T_STAGES;
    uint64_t* acc_bar = empty_bar + T_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* rp = reinterpret_cast<int*>(tmem_slot + 2);            // [PANEL_ROWS + 1]
    uint32_t* chunk_mask = reinterpret_cast<uint32_t*>(rp + 12);  // [nchunk]
    int* tile_at = reinterpret_cast<int*>(chunk_mask + ((nchunk + 3) & ~3));  // [8][nbc]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int panel = blockIdx.x;
    const int m0 = blockIdx.y * TBM;
    const int nbr = out >> 4;

    // ---- prologue: panel index tables ----
    if (threadIdx.x <= PANEL_ROWS) {
        int br = panel * PANEL_ROWS + threadIdx.x;
        br = br < nbr ? br : nbr;
        rp[threadIdx.x] = __ldg(row_ptr + br);
    }
    for (int i = threadIdx.x; i < nchunk; i += TILE_THREADS) chunk_mask[i] = 0u;
    if (threadIdx.x == 0) {
        for (int s = 0; s < T_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
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
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int panel_tiles = rp[PANEL_ROWS] - rp[0];
    pdl_launch_dependents();
    pdl_wait();  // the index tables above are weights; activations and Y need the wait

    if (warp == 0) {
        // ---------------- producer (whole warp: lane = row * 4 + column in chunk) ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmX);
            tma_prefetch_desc(&tmW);
        }
        const int r = lane >> 2, kb = lane & 3;
        int stage_it = 0;
        bool ok = true;
        for (int kc = 0; kc < nchunk && ok; ++kc) {
            const uint32_t mask = chunk_mask[kc];
            if (mask == 0u) continue;
            const int s = stage_it % T_STAGES;
            const uint32_t ph = (stage_it / T_STAGES) & 1;
            if (lane == 0) {
                ok = mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag);
                if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_PRODUCER);
                else
                    mbar_arrive_expect_tx(&full_bar[s], X_STAGE_BYTES + 512u * __popc(mask));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) tma_load_2d(sX + s * X_STAGE_BYTES, &tmX, &full_bar[s], kc * CHUNK, m0);
            if (mask & (1u << lane)) {
                const int t = tile_at[r * nbc + kc * 4 + kb];
                tma_load_2d(sW + s * W_STAGE_BYTES + lane * 512, &tmW, &full_bar[s], 0, t * 16);
            }
            ++stage_it;
        }
        if (*abort_flag && lane == 0) {
            const int first = stage_it > T_STAGES ? stage_it - T_STAGES : 0;
            for (int it2 = first; it2 < stage_it; ++it2)
                for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                    if (mbar_try_wait(&full_bar[it2 % T_STAGES], (it2 / T_STAGES) & 1)) break;
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
                const int s = stage_it % T_STAGES;
                const uint32_t ph = (stage_it / T_STAGES) & 1;
                if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t x_addr = smem_u32(sX + s * X_STAGE_BYTES);
                const uint32_t w_addr = smem_u32(sW + s * W_STAGE_BYTES);
                while (mask) {
                    const int bit = __ffs(mask) - 1;
                    mask &= mask - 1;
                    const int r = bit >> 2, kb = bit & 3;
                    const uint64_t ad = make_smem_desc(x_addr + kb * 32, 16, 1024, SWZ_128B);
                    const uint64_t bd = make_smem_desc(w_addr + bit * 512, 16, 256, SWZ_32B);
                    mma_f16_ss(tmem_base + r * 16, ad, bd, idesc, (started >> r) & 1u);
                    started |= 1u << r;
                }
                mma_commit(&empty_bar[s]);
                ++stage_it;
            }
            if (ok) mma_commit(acc_bar);
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        bool ok = true;
        if (panel_tiles > 0) {
            ok = mbar_wait_bounded(acc_bar, 0, abort_flag);
            if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_EPILOGUE);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
#pragma unroll 1
            for (int r = 0; r < PANEL_ROWS; ++r) {
                const int col0 = (panel * PANEL_ROWS + r) * 16;
                if (col0 >= out) break;
                uint32_t v[16];
                if (rp[r + 1] > rp[r]) {
                    tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + r * 16, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
                if (row < T) {
                    float f[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
                    if (bias != nullptr) {
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            const uint4 bq = __ldg(reinterpret_cast<const uint4*>(bias + col0 + g * 8));
                            const __half2* bh = reinterpret_cast<const __half2*>(&bq);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 bf = __half22float2(bh[j]);
                                f[g * 8 + 2 * j] += bf.x;
                                f[g * 8 + 2 * j + 1] += bf.y;
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) f[j] = apply_act(f[j], act);
                    uint4 o0, o1;
                    o0.x = pack_half2(f[0], f[1]);
                    o0.y = pack_half2(f[2], f[3]);
                    o0.z = pack_half2(f[4], f[5]);
                    o0.w = pack_half2(f[6], f[7]);
                    o1.x = pack_half2(f[8], f[9]);
                    o1.y = pack_half2(f[10], f[11]);
                    o1.z = pack_half2(f[12], f[13]);
                    o1.w = pack_half2(f[14], f[15]);
                    __half* y = Y + static_cast<size_t>(row) * out + col0;
                    *reinterpret_cast<uint4*>(y) = o0;
                    *reinterpret_cast<uint4*>(y + 8) = o1;
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
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

    CUtensorMap tmX, tmW;
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
    const int nbc = in / 16, nchunk = (in + CHUNK - 1) / CHUNK;
    const int smem_bytes = T_STAGES * T_STAGE_BYTES + 256 /*barriers + rp*/ +
                           ((nchunk + 3) & ~3) * 4 + PANEL_ROWS * nbc * 4 + 1024;
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
                         row_ptr, row_off, bias, Y, T, in, out, act, err) == cudaSuccess
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
