// Tile-pruned Linear on re-packed weights, persistent form.
//
// One CTA per SM walks a list of work items (128 tokens x 2 panels of 8 output block rows =
// 256 output features).  What a 16 x 16 weight tile costs on this tensor core is fixed by the
// instruction, not by its arithmetic: a 128 x 16 x 16 tcgen05.mma occupies the pipe 39 cycles
// when products are issued from several threads, 60 from one (measured), whatever operand
// feeds it.  So the kernel is built to keep the pipe issuing and to pay nothing else per tile:
//   * warp 0 streams, per 64-feature chunk that holds any tile of the item, the 128 x 64
//     activation slab (tiled bulk copy, 128-byte swizzle) and the chunk's tiles of both panels
//     (two untiled bulk copies of pre-swizzled tiles) through a ring of 3-5 stages;
//   * warps 2-9: one thread each issues the products of block row (warp - 2) of both panels
//     and commits them to the stage's barrier, so eight threads feed the pipe in parallel;
//   * warps 10-17 drain the PREVIOUS item's accumulators (tensor memory holds two items'
//     worth, 2 x 256 columns) - bias, activation, fp16, swizzled staging tile, bulk store -
//     while the current item's products run, and item boundaries cost no pipeline drain;
//   * chunk masks / tile offsets are read straight from the packed arrays, 32 chunks per
//     warp-wide load, and handed to the working lane by shuffles; nothing per item is staged
//     in shared memory, no per-item block-wide barrier exists.
// Every wait is bounded; a wait that runs out records a code and the CTA drains and returns.
#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

constexpr int P_TBM = 128;          // tokens per item
constexpr int P_ROWS = 8;           // block rows per panel
constexpr int P_PANELS = 2;         // panels per item
constexpr int P_TBN = P_ROWS * 16;  // output features per panel
constexpr int P_CHUNK = 64;         // input features per ring stage
constexpr int P_X_BYTES = P_TBM * P_CHUNK * 2;
constexpr int P_RING_BYTES = 160 * 1024;
constexpr int P_MAX_STAGES = 5;
constexpr int P_ISSUERS = 8;
constexpr int P_EPI_WARPS = 8;
constexpr int P_THREADS = 32 * (2 + P_ISSUERS + P_EPI_WARPS);
constexpr int P_STAGING_BYTES = P_EPI_WARPS * 4096;
constexpr int P_MISC_BYTES = 1024;
constexpr int P_SMEM_BYTES = P_RING_BYTES + P_STAGING_BYTES + P_MISC_BYTES + 1024;

struct TileItem {
    int m0;      // first token
    int panel0;  // first of the two panels
};

template <int ACT>
__global__ void __launch_bounds__(P_THREADS, 1)
linear_tile_persist_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                           const uint32_t* __restrict__ pk_mask,
                           const int* __restrict__ pk_off, const __half* __restrict__ pk_tiles,
                           const __half* __restrict__ bias, int T, int in, int out, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* ring = smem;
    uint8_t* staging = smem + P_RING_BYTES;
    uint8_t* misc = staging + P_STAGING_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);  // [P_MAX_STAGES]
    uint64_t* empty_bar = full_bar + P_MAX_STAGES;           // [P_MAX_STAGES]
    uint64_t* acc_full = empty_bar + P_MAX_STAGES;           // [2]
    uint64_t* acc_empty = acc_full + 2;                      // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* max_cnt = reinterpret_cast<int*>(tmem_slot + 2);
    float* s_bias = reinterpret_cast<float*>(misc + 256);  // [P_EPI_WARPS][64]: a warp's columns

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nchunk = (in + P_CHUNK - 1) / P_CHUNK;
    const int ngroup = (nchunk + 31) >> 5;  // groups of 32 chunks (one warp-wide load each)
    const int nbr = out >> 4;
    const int npanel = (out + P_TBN - 1) / P_TBN;
    const int items_n = (npanel + P_PANELS - 1) / P_PANELS;
    const int items_m = (T + P_TBM - 1) / P_TBM;
    const int total_items = items_n * items_m;
    // consecutive items share a token block: CTAs that run side by side read the same
    // activation rows from L2
    auto item_of = [&](int t) {
        TileItem it;
        it.m0 = (t / items_n) * P_TBM;
        it.panel0 = (t % items_n) * P_PANELS;
        return it;
    };

    // ---- set-up (weights only: may overlap the previous kernel's tail) ----
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmY);
        for (int s = 0; s < P_MAX_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], P_ISSUERS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], P_ISSUERS);
            mbar_init(&acc_empty[b], P_EPI_WARPS);
        }
        *abort_flag = 0;
        *max_cnt = 1;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    __syncthreads();
    {
        // the ring's stage size follows the fullest (panel, chunk) of the whole weight
        int mc = 0;
        for (int i = threadIdx.x; i < npanel * nchunk; i += P_THREADS) {
            const int cnt = __popc(__ldg(pk_mask + i));
            mc = cnt > mc ? cnt : mc;
        }
        for (int d = 16; d > 0; d >>= 1) {
            const int o = __shfl_xor_sync(0xffffffffu, mc, d);
            mc = o > mc ? o : mc;
        }
        if (lane == 0 && mc > 1) atomicMax(max_cnt, mc);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int nslot = (*max_cnt + 3) & ~3;  // tile slots per panel and stage
    const int stage_bytes = P_X_BYTES + P_PANELS * nslot * 512;
    const int nstages =
        P_RING_BYTES / stage_bytes < P_MAX_STAGES ? P_RING_BYTES / stage_bytes : P_MAX_STAGES;
    pdl_launch_dependents();
    pdl_wait();  // activations and Y belong to the kernels before / after this one

    // the masks of 32 chunks (chunk = group * 32 + lane) of the item's two panels
    auto load_masks = [&](const TileItem& it, int g, uint32_t& m0, uint32_t& m1) {
        const int c = g * 32 + lane;
        m0 = m1 = 0u;
        if (c < nchunk) {
            if (it.panel0 < npanel) m0 = __ldg(pk_mask + static_cast<size_t>(it.panel0) * nchunk + c);
            if (it.panel0 + 1 < npanel)
                m1 = __ldg(pk_mask + static_cast<size_t>(it.panel0 + 1) * nchunk + c);
        }
    };

    if (warp == 0) {
        // ---------------- producer ----------------
        int s = 0, issued = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
            const TileItem it = item_of(t);
            for (int g = 0; g < ngroup && ok; ++g) {
                uint32_t m0, m1;
                load_masks(it, g, m0, m1);
                const int c = g * 32 + lane;
                int o0 = 0, o1 = 0;
                if (m0) o0 = __ldg(pk_off + static_cast<size_t>(it.panel0) * nchunk + c);
                if (m1) o1 = __ldg(pk_off + static_cast<size_t>(it.panel0 + 1) * nchunk + c);
                uint32_t live = __ballot_sync(0xffffffffu, (m0 | m1) != 0u);
                while (live) {
                    const int cc = __ffs(live) - 1;
                    live &= live - 1;
                    const uint32_t mm0 = __shfl_sync(0xffffffffu, m0, cc);
                    const uint32_t mm1 = __shfl_sync(0xffffffffu, m1, cc);
                    const int oo0 = __shfl_sync(0xffffffffu, o0, cc);
                    const int oo1 = __shfl_sync(0xffffffffu, o1, cc);
                    if (lane == 0) {
                        uint8_t* stage = ring + s * stage_bytes;
                        ok = mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag);
                        if (!ok) {
                            report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_PRODUCER);
                        } else {
                            const uint32_t n0 = __popc(mm0), n1 = __popc(mm1);
                            mbar_arrive_expect_tx(&full_bar[s], P_X_BYTES + 512u * (n0 + n1));
                            tma_load_2d(stage, &tmX, &full_bar[s], (g * 32 + cc) * P_CHUNK, it.m0);
                            if (n0)
                                bulk_load(stage + P_X_BYTES, pk_tiles + static_cast<size_t>(oo0) * 256,
                                          512u * n0, &full_bar[s]);
                            if (n1)
                                bulk_load(stage + P_X_BYTES + nslot * 512,
                                          pk_tiles + static_cast<size_t>(oo1) * 256, 512u * n1,
                                          &full_bar[s]);
                            ++issued;
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
        if (*abort_flag && lane == 0) {
            // let copies in flight land: the last min(issued, nstages) stages
            int ss = s;
            uint32_t pp = ph;
            const int pending = issued < nstages ? issued : nstages;
            for (int i = 0; i < pending; ++i) {
                if (--ss < 0) {
                    ss = nstages - 1;
                    pp ^= 1u;
                }
                for (uint32_t k = 0; k < ET_SPIN_LIMIT; ++k)
                    if (mbar_try_wait(&full_bar[ss], pp)) break;
            }
        }
    } else if (warp >= 2 && warp < 2 + P_ISSUERS) {
        // ---------------- product issue: block row e of both panels ----------------
        const int e = warp - 2;
        constexpr uint32_t idesc = make_idesc_f16(P_TBM, 16, 0, 0);
        const uint32_t ring_addr = smem_u32(ring);
        // descriptors differ between stages and tiles only in the start-address field (16-byte
        // units)
        const uint64_t a_desc0 = make_smem_desc(ring_addr, 16, 1024, SWZ_128B);
        const uint64_t b_desc0 = make_smem_desc(ring_addr + P_X_BYTES, 16, 256, SWZ_32B);
        const uint32_t stage_units = static_cast<uint32_t>(stage_bytes) >> 4;
        const uint32_t panel_units = static_cast<uint32_t>(nslot) * 32u;
        const uint32_t below = (1u << (4 * e)) - 1u;
        int s = 0, item_it = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x, ++item_it) {
            const TileItem it = item_of(t);
            const int buf = item_it & 1;
            if (item_it >= 2) {
                // the epilogue must have drained what the item two back left in this buffer
                if (lane == 0) {
                    ok = mbar_wait_bounded(&acc_empty[buf], ((item_it >> 1) - 1) & 1, abort_flag);
                    if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                tc_fence_after_sync();
            }
            const uint32_t d_tmem = tmem_base + buf * (P_PANELS * P_TBN) + e * 16;
            uint32_t started = 0u;  // bit j: this row of panel j has received a product
            for (int g = 0; g < ngroup && ok; ++g) {
                uint32_t m0, m1;
                load_masks(it, g, m0, m1);
                // per chunk: bits 0-3 the row's tiles among the chunk's 4 block columns, bits 4-9
                // the row's first slot among the panel's tiles of the chunk
                const uint32_t c0 = ((m0 >> (4 * e)) & 0xFu) | (__popc(m0 & below) << 4);
                const uint32_t c1 = ((m1 >> (4 * e)) & 0xFu) | (__popc(m1 & below) << 4);
                uint32_t live = __ballot_sync(0xffffffffu, (m0 | m1) != 0u);
                while (live) {
                    const int cc = __ffs(live) - 1;
                    live &= live - 1;
                    const uint32_t cmd0 = __shfl_sync(0xffffffffu, c0, cc);
                    const uint32_t cmd1 = __shfl_sync(0xffffffffu, c1, cc);
                    if (lane == 0) {
                        // a row without a tile in this chunk still waits: its arrival must not
                        // run ahead into the stage's next use
                        ok = mbar_wait_bounded(&full_bar[s], ph, abort_flag);
                        if (!ok) {
                            report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                        } else if ((cmd0 | cmd1) & 0xFu) {
                            tc_fence_after_sync();
                            const uint64_t a_base = a_desc0 + static_cast<uint64_t>(s) * stage_units;
                            const uint64_t b_base = b_desc0 + static_cast<uint64_t>(s) * stage_units;
#pragma unroll
                            for (int j = 0; j < P_PANELS; ++j) {
                                const uint32_t cmd = j == 0 ? cmd0 : cmd1;
                                uint32_t nib = cmd & 0xFu;
                                uint64_t bd = b_base + j * panel_units + ((cmd >> 4) & 0x3Fu) * 32u;
                                while (nib) {
                                    const int kb = __ffs(nib) - 1;
                                    nib &= nib - 1;
                                    mma_f16_ss(d_tmem + j * P_TBN, a_base + static_cast<uint64_t>(kb * 2),
                                               bd, idesc, (started >> j) & 1u);
                                    started |= 1u << j;
                                    bd += 32;  // next 512-byte slot
                                }
                            }
                            mma_commit(&empty_bar[s]);
                        } else {
                            mbar_arrive(&empty_bar[s]);
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (ok && lane == 0) mma_commit(&acc_full[buf]);  // arrives once this row's products are done
        }
    } else if (warp >= 2 + P_ISSUERS) {
        // ---------------- epilogue: bias, activation, fp16, store ----------------
        const int w = warp - (2 + P_ISSUERS);  // 0 .. 7
        const int q = warp & 3;                // tensor-memory lane quadrant this warp may read
        const int half = w >> 2;               // which 64 output columns of each panel
        uint8_t* tile = staging + w * 4096;
        uint8_t* srow = tile + lane * 128;
        float* wb = s_bias + w * 64;
        bool ok = true;
        bool stored = false;
        int item_it = 0;
        for (int t = blockIdx.x; t < total_items; t += gridDim.x, ++item_it) {
            const TileItem it = item_of(t);
            const int buf = item_it & 1;
            // which block rows of the two panels hold any tile at all: rows without one were
            // never written by the tensor core and carry the bias alone
            uint32_t any0 = 0u, any1 = 0u;
            for (int g = 0; g < ngroup; ++g) {
                uint32_t m0, m1;
                load_masks(it, g, m0, m1);
                any0 |= m0;
                any1 |= m1;
            }
            for (int d = 16; d > 0; d >>= 1) {
                any0 |= __shfl_xor_sync(0xffffffffu, any0, d);
                any1 |= __shfl_xor_sync(0xffffffffu, any1, d);
            }
            if (ok) {
                ok = mbar_wait_bounded_relaxed(&acc_full[buf], (item_it >> 1) & 1, abort_flag);
                if (!ok && lane == 0) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_EPILOGUE);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;
            tc_fence_after_sync();
#pragma unroll
            for (int k = 0; k < P_PANELS; ++k) {
                const int n0 = (it.panel0 + k) * P_TBN + half * 64;
                if (n0 >= out) continue;
                const uint32_t anyk = k == 0 ? any0 : any1;
                // this warp's 64 bias values (private to the warp: no block-wide barrier)
                if (stored) {
                    if (lane == 0) tma_store_wait_read();  // the staging tile is free again
                    __syncwarp();
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int n = n0 + lane + 32 * i;
                    wb[lane + 32 * i] = (bias != nullptr && n < out) ? __half2float(__ldg(bias + n)) : 0.f;
                }
                __syncwarp();
                const uint32_t lane_addr = tmem_base + buf * (P_PANELS * P_TBN) + k * P_TBN + half * 64 +
                                           (static_cast<uint32_t>(q * 32) << 16);
                uint32_t v0[32], v1[32];
                tmem_ld32(lane_addr, v0);
                tmem_ld32(lane_addr + 32, v1);
                tmem_ld_wait();
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    // 32 columns = block rows 2 * (half * 2 + cc) and the next of the panel
                    const int br = (half * 2 + cc) * 2;
                    const bool has0 = ((anyk >> (4 * br)) & 0xFu) != 0u;
                    const bool has1 = ((anyk >> (4 * (br + 1))) & 0xFu) != 0u;
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) {
                        float f[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t raw = cc == 0 ? v0[gq * 8 + j] : v1[gq * 8 + j];
                            const bool has = gq < 2 ? has0 : has1;
                            f[j] = apply_act((has ? __uint_as_float(raw) : 0.f) + wb[cc * 32 + gq * 8 + j],
                                             ACT);
                        }
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
                if (lane == 0 && it.m0 + q * 32 < T) {
                    tma_store_2d(&tmY, tile, n0, it.m0 + q * 32);
                    tma_store_commit();
                }
                stored = true;
            }
            // the accumulators of this buffer have been read: the item after next may overwrite them
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (stored && lane == 0) tma_store_wait_read();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

int g_tile_persist = 1;  // test hook: 0 = the one-item-per-CTA kernel for packed weights too

bool tile_persist_enabled() { return g_tile_persist != 0; }

int launch_linear_tile_persist(const int* row_ptr, const uint32_t* pk_mask, const int* pk_off,
                               const __half* pk_tiles, int nnz_tiles, const __half* bias,
                               const __half* X, __half* Y, int T, int in, int out, int act,
                               cudaStream_t stream) {
    if (!row_ptr || !pk_mask || !pk_off || !pk_tiles || !X || !Y || T <= 0 || in <= 0 || out <= 0 ||
        nnz_tiles <= 0)
        return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16 || in > 8192) return ET_ERR_SHAPE;
    if (!aligned16(X) || !aligned16(Y) || !aligned16(pk_tiles) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;
    CUtensorMap tmX, tmY;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(in), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(in) * 2};
        const uint32_t box[2] = {P_CHUNK, P_TBM};
        int st = make_tensor_map_f16(&tmX, X, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(out), static_cast<uint64_t>(T)};
        const uint64_t strides[1] = {static_cast<uint64_t>(out) * 2};
        const uint32_t box[2] = {64, 32};
        int st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    const int npanel = (out + P_TBN - 1) / P_TBN;
    const int items = ((npanel + P_PANELS - 1) / P_PANELS) * ((T + P_TBM - 1) / P_TBM);
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const dim3 grid(items < sms ? items : sms);
    int dev = 0;
    cudaGetDevice(&dev);
    auto go = [&](auto kern, int slot) -> cudaError_t {
        static std::atomic<bool> attr_set[3][64] = {};
        if (dev >= 0 && dev < 64 && !attr_set[slot][dev]) {
            const cudaError_t ea =
                cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
            if (ea != cudaSuccess) return ea;
            attr_set[slot][dev] = true;
        }
        return launch_kernel(kern, grid, dim3(P_THREADS), P_SMEM_BYTES, stream, tmX, tmY, pk_mask,
                             pk_off, pk_tiles, bias, T, in, out, err);
    };
    const cudaError_t e = act == ET_ACT_GELU   ? go(linear_tile_persist_kernel<ET_ACT_GELU>, 0)
                          : act == ET_ACT_RELU ? go(linear_tile_persist_kernel<ET_ACT_RELU>, 1)
                                               : go(linear_tile_persist_kernel<ET_ACT_NONE>, 2);
    return e == cudaSuccess ? ET_OK : ET_ERR_CUDA;
}

}  // namespace et

#ifdef ET_TEST_HOOKS
extern "C" {
// Test hook: 1 = persistent kernel for packed weights (default), 0 = one item per CTA.
void et_debug_set_tile_persist(int on) { et::g_tile_persist = on; }
}
#endif
