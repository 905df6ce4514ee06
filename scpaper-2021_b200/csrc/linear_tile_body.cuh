// Body of the tile-pruned Linear kernel for one (128-token block, panel of output block rows),
// shared by the stand-alone kernels (linear_tile.cu) and the attention kernel that also runs the
// output projection (attention_fuse_o.cu).
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
//
// Packed form.  Issuing one TMA per 512-byte tile makes the producer the bottleneck at high
// sparsity, so the operator can re-pack its (static) weights once: tiles are reordered into
// (pair of panels, chunk, panel, row, column) order - the order in which the kernels consume them - and
// stored pre-swizzled, with one presence mask and one tile offset per (panel, chunk).  A
// chunk's tiles are then one contiguous run fetched by a single bulk copy, and the prologue
// reads ready-made masks instead of building them.  The re-packing is a pure permutation of
// the tile-CSR arrays (et_tile_pack_plan on the host indices, et_tile_pack_tiles on the GPU).
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace et {
namespace tile {

// Optional per-CTA timestamps for bring-up builds (-DET_TIMELINE); compiled out otherwise.
#undef ET_TL
#ifdef ET_TIMELINE
static __device__ long long et_tile_timeline[4096];
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

// PACKED: pk_mask / pk_off / tiles describe the re-packed weights (row_off unused).
// ACT: the activation, compiled in.  NP: panels of 8 output block rows per CTA (1, or 2 for
// packed weights with many panels: both panels share every activation slab, which halves the
// activation traffic and the per-CTA fixed cost per output).
//
// The work of one CTA: tokens [m0, m0 + 128) x panels [panel0, panel0 + NP).  `smem` is the
// CTA's 1024-byte-aligned dynamic shared memory.
// FUSED == false: the body of a kernel of its own - it allocates and frees tensor memory, owns
// the abort flag and takes part in programmatic dependent launch.
// FUSED == true: one of several pieces of work a CTA runs in turn - tensor memory (tmem_in) and
// the abort flag (abort_in) belong to the caller, the activations may have been written by
// other CTAs of the same grid - wait_inputs(), called by every thread once the index tables
// (weights only) are built, returns when they are complete - and the barriers are invalidated
// at the end so that the next piece of work may lay out shared memory afresh.
struct NoInputWait {
    __device__ __forceinline__ void operator()() const {}
};
template <bool PACKED, int ACT, int NP, bool FUSED, typename WaitFn = NoInputWait>
__device__ __forceinline__ void linear_tile_cta(
    const CUtensorMap& tmX, const CUtensorMap& tmW, const CUtensorMap& tmY,
    const int* __restrict__ row_ptr, const int* __restrict__ row_off,
    const uint32_t* __restrict__ pk_mask, const int* __restrict__ pk_off,
    const __half* __restrict__ pk_tiles, const __half* __restrict__ bias, int T, int in, int out,
    int* err_word, uint8_t* smem, int panel0, int m0, uint32_t tmem_in, volatile int* abort_in,
    WaitFn wait_inputs = WaitFn()) {
    static_assert(NP == 1 || PACKED, "two panels per CTA exist for packed weights only");
    const int nbc = in >> 4;  // input block columns
    const int nchunk = (in + CHUNK - 1) / CHUNK;
    const int nchunk_p = (nchunk + 3) & ~3;
    uint8_t* ring = smem;
    uint8_t* misc = smem + RING_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
    uint64_t* empty_bar = full_bar + MAX_STAGES;
    uint64_t* acc_bar = empty_bar + MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = FUSED ? abort_in : reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* max_cnt = reinterpret_cast<int*>(tmem_slot + 2);
    int* rp = reinterpret_cast<int*>(tmem_slot + 4);                       // [NP][PANEL_ROWS + 1]
    float* s_bias = reinterpret_cast<float*>(misc + 256);                  // [NP * TBN]
    uint32_t* chunk_mask = reinterpret_cast<uint32_t*>(s_bias + NP * TBN);  // [NP][nchunk_p]
    // unpacked: tile_at[8][nbc]; packed: [NP][nchunk_p] (first tile of each chunk)
    int* tile_at = reinterpret_cast<int*>(chunk_mask + NP * nchunk_p);
    // per (panel, block row) and chunk, what the issuing thread of that row needs: bits 0-3
    // which of the chunk's 4 block columns hold a tile of the row, bits 4-9 the row's first
    // slot among the panel's tiles of the chunk, bit 15 set when the whole CTA skips the chunk
    uint16_t* cmd = reinterpret_cast<uint16_t*>(tile_at + (PACKED ? NP * nchunk_p : PANEL_ROWS * nbc));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nbr = out >> 4;
    const int npanel = (out + TBN - 1) / TBN;

    // ---- prologue: panel index tables and bias (weights: independent of earlier kernels) ----
    if (threadIdx.x == 0) ET_TL(0);
    if (threadIdx.x < NP * (PANEL_ROWS + 1)) {
        const int k = threadIdx.x / (PANEL_ROWS + 1), i = threadIdx.x % (PANEL_ROWS + 1);
        int br = (panel0 + k) * PANEL_ROWS + i;
        br = br < nbr ? br : nbr;
        rp[threadIdx.x] = __ldg(row_ptr + br);
    }
    for (int i = threadIdx.x; i < NP * nchunk; i += TILE_THREADS) {
        const int k = i / nchunk, c = i - k * nchunk;
        if (PACKED) {
            const bool live = panel0 + k < npanel;
            chunk_mask[k * nchunk_p + c] =
                live ? __ldg(pk_mask + static_cast<size_t>(panel0 + k) * nchunk + c) : 0u;
            tile_at[k * nchunk_p + c] =
                live ? __ldg(pk_off + static_cast<size_t>(panel0 + k) * nchunk + c) : 0;
        } else {
            chunk_mask[c] = 0u;
        }
    }
    for (int i = threadIdx.x; i < NP * TBN; i += TILE_THREADS) {
        const int n = panel0 * TBN + i;
        s_bias[i] = (bias != nullptr && n < out) ? __half2float(__ldg(bias + n)) : 0.f;
    }
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmW);
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], T_EPI_WARPS);
        }
        mbar_init(acc_bar, T_EPI_WARPS);
        if (!FUSED) *abort_flag = 0;
        *max_cnt = 0;
        fence_barrier_init();
    }
    if (!FUSED && warp == 1) {
        tmem_alloc(tmem_slot, NP * TBN);
        tmem_relinquish();
    }
    __syncthreads();
    if (!PACKED) {
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
    }
    {
        int mc = 0;
        for (int i = threadIdx.x; i < NP * nchunk; i += TILE_THREADS) {
            const int k = i / nchunk, c = i - k * nchunk;
            const int cnt = __popc(chunk_mask[k * nchunk_p + c]);
            mc = cnt > mc ? cnt : mc;
        }
        if (mc > 0) atomicMax(max_cnt, mc);
        for (int i = threadIdx.x; i < NP * PANEL_ROWS * nchunk; i += TILE_THREADS) {
            const int kr = i / nchunk, c = i - kr * nchunk;
            const int k = kr / PANEL_ROWS, r = kr - k * PANEL_ROWS;
            uint32_t any = 0;
#pragma unroll
            for (int kk = 0; kk < NP; ++kk) any |= chunk_mask[kk * nchunk_p + c];
            const uint32_t m = chunk_mask[k * nchunk_p + c];
            cmd[kr * nchunk_p + c] = static_cast<uint16_t>(
                ((m >> (4 * r)) & 0xFu) | (__popc(m & ((1u << (4 * r)) - 1u)) << 4) |
                (any == 0u ? 0x8000u : 0u));
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = FUSED ? tmem_in : *tmem_slot;
    int panel_tiles = 0;
#pragma unroll
    for (int k = 0; k < NP; ++k)
        panel_tiles += rp[k * (PANEL_ROWS + 1) + PANEL_ROWS] - rp[k * (PANEL_ROWS + 1)];
    // stage geometry: activation slab + densely packed tile slots (per panel)
    const int nslot = *max_cnt <= 16 ? 16 : 32;
    const int stage_bytes = X_STAGE_BYTES + NP * nslot * 512;
    const int nstages = RING_BYTES / stage_bytes;  // 4, 3 or 2
    if (threadIdx.x == 0) ET_TL(1);
    if (!FUSED) {
        pdl_launch_dependents();
        pdl_wait();  // the tables above are weights; activations and Y need the wait
    } else {
        wait_inputs();
    }

    // all panels' masks of one chunk
    auto masks_of = [&](int kc, uint32_t (&m)[NP]) -> uint32_t {
        uint32_t any = 0;
#pragma unroll
        for (int k = 0; k < NP; ++k) {
            m[k] = chunk_mask[k * nchunk_p + kc];
            any |= m[k];
        }
        return any;
    };

    if (warp < 2) {
        // ---------------- producers ----------------
        // packed: lane 0 of warps 0 and 1 take alternate chunks, each fetching the activation
        // slab and the chunk's tiles (one bulk copy per panel); tile-CSR: warp 0 alone, lane =
        // row * 4 + column in chunk fetches its own tile.  Stage index and phase advance
        // incrementally (no divisions on the path).
        int s = 0, issued = 0;
        uint32_t ph = 0;
        // activations written by other CTAs of this grid: the acquire in wait_inputs() comes
        // before the TMA reads of the threads that fetch activation slabs
        if (FUSED && lane == 0) fence_proxy_async_global();
        if (PACKED) {
            if (lane == 0) {
                for (int kc = 0; kc < nchunk; ++kc) {
                    uint32_t m[NP];
                    if (masks_of(kc, m) == 0u) continue;
                    if ((issued & 1) == warp) {
                        uint8_t* stage = ring + s * stage_bytes;
                        if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                            report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_PRODUCER);
                            break;
                        }
                        uint32_t bytes = 0;
#pragma unroll
                        for (int k = 0; k < NP; ++k) bytes += 512u * __popc(m[k]);
                        mbar_arrive_expect_tx(&full_bar[s], X_STAGE_BYTES + bytes);
                        if (issued < 12) ET_TL(16 + issued * 4);
                        tma_load_2d(stage, &tmX, &full_bar[s], kc * CHUNK, m0);
                        // a panel's tiles of the chunk are one contiguous, pre-swizzled run
#pragma unroll
                        for (int k = 0; k < NP; ++k)
                            if (m[k] != 0u)
                                bulk_load(stage + X_STAGE_BYTES + k * nslot * 512,
                                          pk_tiles + static_cast<size_t>(tile_at[k * nchunk_p + kc]) * 256,
                                          512u * __popc(m[k]), &full_bar[s]);
                        if (issued < 12) ET_TL(17 + issued * 4);
                    }
                    ++issued;
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        } else if (warp == 0) {
            const int r = lane >> 2, kb = lane & 3;
            bool ok = true;
            for (int kc = 0; kc < nchunk && ok; ++kc) {
                const uint32_t mask = chunk_mask[kc];
                if (mask == 0u) continue;
                uint8_t* stage = ring + s * stage_bytes;
                if (lane == 0) {
                    ok = mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag);
                    if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_PRODUCER);
                    else
                        mbar_arrive_expect_tx(&full_bar[s], X_STAGE_BYTES + 512u * __popc(mask));
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (lane == 0) tma_load_2d(stage, &tmX, &full_bar[s], kc * CHUNK, m0);
                if (mask & (1u << lane)) {
                    const int t = tile_at[r * nbc + kc * 4 + kb];
                    const int slot = __popc(mask & ((1u << lane) - 1u));
                    tma_load_2d(stage + X_STAGE_BYTES + slot * 512, &tmW, &full_bar[s], 0, t * 16);
                }
                ++issued;
                if (++s == nstages) {
                    s = 0;
                    ph ^= 1u;
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
                for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                    if (mbar_try_wait(&full_bar[ss], pp)) break;
            }
        }
    } else {
        // ------- warps 2..9: MMA issue for one block row (of every panel) each, then the epilogue
        // Issuing a 128 x 16 x 16 product costs far more issue time than tensor time, so the
        // eight block rows of a panel are issued by eight threads in parallel; every warp
        // commits its own products to the stage's empty barrier and to the accumulator barrier.
        const int e = warp - 2;            // block row issued by this warp
        const int q = warp & 3;            // TMEM lane quadrant read in the epilogue
        const int half = (warp - 2) >> 2;  // which 64 output columns of a panel
        bool ok = true;
        if (panel_tiles > 0) {
            // one thread per warp issues: warp e owns block row e of every panel (accumulator
            // rows e, e + 8, ...) and reads those rows' per-chunk commands
            if (lane == 0) {
                constexpr uint32_t idesc = make_idesc_f16(TBM, 16, 0, 0);
                uint32_t started = 0u;  // bit j: this warp's row of panel j has received a product
                int s = 0, stage_it = 0;
                uint32_t ph = 0;
                const uint32_t ring_addr = smem_u32(ring);
                // descriptors differ from stage to stage and tile to tile only in their start
                // address field (16-byte units)
                const uint64_t a_desc0 = make_smem_desc(ring_addr, 16, 1024, SWZ_128B);
                const uint64_t b_desc0 = make_smem_desc(ring_addr + X_STAGE_BYTES, 16, 256, SWZ_32B);
                const uint32_t stage_units = static_cast<uint32_t>(stage_bytes) >> 4;
                const uint32_t panel_units = static_cast<uint32_t>(nslot) * 32u;
                for (int kc = 0; kc < nchunk; ++kc) {
                    uint32_t c[NP];
                    uint32_t any = 0u;
#pragma unroll
                    for (int j = 0; j < NP; ++j) {
                        c[j] = cmd[(j * PANEL_ROWS + e) * nchunk_p + kc];
                        any |= c[j] & 0xFu;
                    }
                    if (c[0] & 0x8000u) continue;
                    // a warp without a tile in this chunk still waits: its arrival must not
                    // run ahead into the stage's next use
                    if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                        report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_MMA);
                        ok = false;
                        break;
                    }
                    if (e == 0 && stage_it < 12) ET_TL(18 + stage_it * 4);
                    if (any) {
                        tc_fence_after_sync();
                        const uint64_t a_base = a_desc0 + static_cast<uint64_t>(s) * stage_units;
                        const uint64_t b_base = b_desc0 + static_cast<uint64_t>(s) * stage_units;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            uint32_t nib = c[j] & 0xFu;
                            if (nib == 0u) continue;
                            uint64_t bd = b_base + j * panel_units + ((c[j] >> 4) & 0x3Fu) * 32u;
                            while (nib) {
                                const int kb = __ffs(nib) - 1;
                                nib &= nib - 1;
                                mma_f16_ss(tmem_base + j * TBN + e * 16,
                                           a_base + static_cast<uint64_t>(kb * 2), bd, idesc,
                                           (started >> j) & 1u);
                                started |= 1u << j;
                                bd += 32;  // next 512-byte slot
                            }
                        }
                        mma_commit(&empty_bar[s]);
                    } else {
                        mbar_arrive(&empty_bar[s]);
                    }
                    if (e == 0 && stage_it < 12) ET_TL(19 + stage_it * 4);
                    ++stage_it;
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) mma_commit(acc_bar);
                if (e == 0) ET_TL(2);
            }
            __syncwarp();
            ok = mbar_wait_bounded(acc_bar, 0, abort_flag);
            if (!ok && lane == 0) report_error(err_word, abort_flag, DEV_TIMEOUT_TILE_EPILOGUE);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (threadIdx.x == 64) ET_TL(3);
        bool stored = false;
#pragma unroll
        for (int k = 0; k < NP; ++k) {
            const int n0 = (panel0 + k) * TBN;
            if (!ok || n0 + half * 64 >= out) continue;
            tc_fence_after_sync();
            const int* rpk = rp + k * (PANEL_ROWS + 1);
            const bool panel_has_tiles = rpk[PANEL_ROWS] > rpk[0];
            // every MMA has completed: the ring is idle and serves as the staging area
            uint8_t* tile = ring + (k * 8 + q * 2 + half) * 4096;
            uint8_t* srow = tile + lane * 128;
            const uint32_t lane_addr = tmem_base + k * TBN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = half * 2 + cc;  // 32-column chunk = block rows 2c, 2c + 1
                uint32_t v[32];
                if (panel_has_tiles) {
                    tmem_ld32(lane_addr + c * 32, v);
                    tmem_ld_wait_regs(v);
                }
                // block rows without a stored tile were never written by the tensor core
                const bool has0 = rpk[2 * c + 1] > rpk[2 * c], has1 = rpk[2 * c + 2] > rpk[2 * c + 1];
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
                        f[j] = apply_act(__uint_as_float(v[gq * 8 + j]) +
                                             s_bias[k * TBN + c * 32 + gq * 8 + j],
                                         ACT);
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
                stored = true;
            }
        }
        if (stored) {
            tma_store_commit();
            tma_store_wait_read();
        }
        if (threadIdx.x == 64) ET_TL(4);
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) ET_TL(5);
    if (FUSED) {
        if (threadIdx.x == 0 && !*abort_flag)
            for (int i = 0; i < 2 * MAX_STAGES + 1; ++i) mbar_inval(full_bar + i);
        __syncthreads();  // nobody reuses this memory while the barriers are still alive
    } else if (warp == 1) {
        tmem_dealloc(tmem_base, NP * TBN);
    }
}

}  // namespace tile
}  // namespace et
