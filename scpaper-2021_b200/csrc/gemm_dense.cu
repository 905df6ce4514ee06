// Dense fp16 GEMM  Y[M, N] = act(X[M, K] . W[N, K]^T + bias)  on tcgen05 tensor cores.
//
// Each CTA walks a static list of 128 x BN output tiles (persistent form: one CTA per SM and
// several tiles each; single-tile form: one tile per CTA, two CTAs per SM).  Warp 0
// streams 128x64 (X) and BNx64 (W) K-major tiles into a ring of 128-byte-swizzled
// shared-memory stages with TMA; one thread of warp 1 issues tcgen05.mma (M=128, N=BN, K=16)
// into one of TWO fp32 accumulators in tensor memory, so that warps 2-9 (two per
// tensor-memory lane quadrant) can drain the accumulator of tile i - software-pipelined
// tcgen05.ld, bias staged in shared memory, activation, fp16, swizzled staging tile, TMA
// store - while the tensor core already works on tile i + 1.  Rows / columns / K beyond the
// problem are zero-filled by TMA on the way in and clipped on the way out.  Every mbarrier
// wait is bounded.
//
// Output modes: fp16 tile store (Linear layers), index-list store (row-pruned Linear:
// scattered or compressed columns), grouped rows (per-head V.O projection), and fp32
// split-K partials (consumed by the partial-sum LayerNorm kernel).
#include <atomic>

#include "common.cuh"
#include "gemm_common.cuh"
#include "kernels.h"

namespace et {

// Bring-up aid: with -DET_TIMELINE every CTA records clock64() at a few points of its life.
#ifdef ET_TIMELINE
__device__ long long et_gemm_timeline[4096 * 16];
#define ET_TL(slot) \
    do { if (blockIdx.x < 4096) et_gemm_timeline[blockIdx.x * 16 + (slot)] = clock64(); } while (0)
#else
#define ET_TL(slot) ((void)0)
#endif

namespace {

using namespace gemm;

// PERSIST: several tiles per CTA, two accumulators, dedicated staging tiles (the ring keeps
// running during the epilogue).  !PERSIST: exactly one tile per CTA, one accumulator, the
// staging tiles reuse the then idle ring, small enough for two CTAs per SM.
template <int BN, int STAGES, bool PERSIST>
struct GemmCfg {
    static constexpr int B_STAGE_BYTES = BN * BK * 2;
    // One tcgen05.mma covers at most 256 columns and one TMA box at most 256 rows: a wider tile
    // is two halves side by side, in shared memory and in the accumulator.
    static constexpr int MMA_N = BN > 256 ? BN / 2 : BN;
    static constexpr int N_HALVES = BN / MMA_N;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    // staging tiles of the epilogue: one 4 KB tile per (quadrant, 64 fp16 columns) or, for fp32
    // partials (BN <= 128 only), per (quadrant, 32 fp32 columns)
    static constexpr int STAGING_NEED = BN <= 128 ? BN * 512 : BN * 256;
    static constexpr int STAGING_BYTES = PERSIST ? STAGING_NEED : 0;
    static constexpr int MISC_BYTES = 256 + 2 * 8 * BN;  // barriers + 2 x (bias fp32 + column ids)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + MISC_BYTES + 1024;
    static constexpr int NACC = PERSIST ? 2 : 1;
    static constexpr int TMEM_NEED = NACC * BN;  // allocations are powers of two, at least 32
    static constexpr int TMEM_COLS = TMEM_NEED <= 32    ? 32
                                     : TMEM_NEED <= 64  ? 64
                                     : TMEM_NEED <= 128 ? 128
                                     : TMEM_NEED <= 256 ? 256
                                                        : 512;
    static constexpr int MIN_CTAS = (!PERSIST && SMEM_BYTES <= 113 * 1024) ? 2 : 1;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget exceeded");
    static_assert(TMEM_NEED <= 512, "tensor memory budget exceeded");
    static_assert(PERSIST || STAGES * STAGE_BYTES >= STAGING_NEED, "staging does not fit the ring");
};

struct TileCoord {
    int n0, m0, z, kb_begin, num_kb;
};

// B_MN == false: W is [N, K] with K contiguous (the Linear weight layout).
// B_MN == true : W is [groups][K, N] with N contiguous; its tiles are consumed in place
//                as MN-major operands (64-column atoms of 64 K-rows, 8 KB each).
// EPI: 0 = every output mode and activation chosen at run time (index-list, grouped and
// partial-sum epilogues); 1 + act = the fp16 tile store with that activation compiled in.  The
// specialised form matters: with all variants inlined behind run-time branches the same
// staging code ran three times slower.
template <int BN, int STAGES, bool PERSIST, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, (GemmCfg<BN, STAGES, PERSIST>::MIN_CTAS))
gemm_f16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmY, const GemmArgs g) {
    using Cfg = GemmCfg<BN, STAGES, PERSIST>;
    const int* __restrict__ col_map = g.col_map;
    const int M = g.M, N = g.N;
    int* err_word = g.err_word;

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    // single-tile form: all MMAs of the tile have completed before the epilogue touches the ring
    uint8_t* sStage = PERSIST ? smem + STAGES * Cfg::STAGE_BYTES : smem;
    uint8_t* misc = smem + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;  // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_bias = reinterpret_cast<float*>(misc + 256);  // [2][BN]
    int* s_col = reinterpret_cast<int*>(s_bias + 2 * BN);  // [2][BN]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_n = (N + BN - 1) / BN;
    const int tiles_m = (M + BM - 1) / BM;
    const int total_tiles = tiles_n * tiles_m * g.nz;
    const int kb_total = (g.K + BK - 1) / BK;

    auto decode = [&](int t) {
        TileCoord c;
        c.n0 = (t % tiles_n) * BN;
        const int rest = t / tiles_n;
        c.m0 = (rest % tiles_m) * BM;
        c.z = rest / tiles_m;
        c.kb_begin = 0;
        int kb_end = kb_total;
        if (g.out_mode == OUT_PARTIAL_F32) {
            c.kb_begin = c.z * g.kb_per_split;
            kb_end = c.kb_begin + g.kb_per_split < kb_total ? c.kb_begin + g.kb_per_split : kb_total;
            if (kb_end < c.kb_begin) kb_end = c.kb_begin;
        }
        c.num_kb = kb_end - c.kb_begin;
        return c;
    };

    if (threadIdx.x == 0) {
        ET_TL(0);
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], EPI_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) ET_TL(1);
    pdl_launch_dependents();  // the next kernel may begin its own set-up

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            int it = 0;  // K blocks issued so far (ring position)
            bool ok = true;
            auto load_b = [&](const TileCoord& c, int kb, int s) {
                if (B_MN) {
#pragma unroll
                    for (int t = 0; t < BN / 64; ++t)
                        tma_load_3d(sB + s * Cfg::B_STAGE_BYTES + t * (BK * 128), &tmB, &full_bar[s],
                                    c.n0 + t * 64, kb * BK, c.z);
                } else {
#pragma unroll
                    for (int h = 0; h < Cfg::N_HALVES; ++h)
                        tma_load_2d(sB + s * Cfg::B_STAGE_BYTES + h * (Cfg::MMA_N * 128), &tmB,
                                    &full_bar[s], kb * BK, c.n0 + h * Cfg::MMA_N);
                }
            };
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const TileCoord c = decode(t);
                int i0 = 0;
                if (t == static_cast<int>(blockIdx.x)) {
                    // Weights do not depend on the previous kernel: fill the ring with weight
                    // tiles first, then wait for the producer of the activations.
                    const int pre = c.num_kb < STAGES ? c.num_kb : STAGES;
                    for (int i = 0; i < pre; ++i) {
                        mbar_arrive_expect_tx(&full_bar[i], Cfg::STAGE_BYTES);
                        load_b(c, c.kb_begin + i, i);
                    }
                    pdl_wait();
                    ET_TL(2);
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d(sA + i * A_STAGE_BYTES, &tmA, &full_bar[i], (c.kb_begin + i) * BK,
                                    c.m0);
                    it = pre;
                    i0 = pre;
                }
                for (int i = i0; i < c.num_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                        report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_PRODUCER);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
                    tma_load_2d(sA + s * A_STAGE_BYTES, &tmA, &full_bar[s], (c.kb_begin + i) * BK,
                                c.m0);
                    load_b(c, c.kb_begin + i, s);
                }
            }
            if (*abort_flag) {
                // Let copies already in flight land before the CTA's shared memory is released.
                const int first = it > STAGES ? it - STAGES : 0;
                for (int i = first; i < it; ++i)
                    for (uint32_t sp = 0; sp < ET_SPIN_LIMIT; ++sp)
                        if (mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(BM, Cfg::MMA_N, 0, B_MN ? 1 : 0);
            int it = 0, tile_iter = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++tile_iter) {
                const TileCoord c = decode(t);
                const int buf = PERSIST ? (tile_iter & 1) : 0;
                const uint32_t use_ph = PERSIST ? ((tile_iter >> 1) & 1) : (tile_iter & 1);
                // (an empty K slice issues no MMA: the commit below then arrives at once and the
                // epilogue writes zeros)
                // the epilogue must have drained this accumulator's previous tile
                if (!mbar_wait_bounded(&acc_empty[buf], use_ph ^ 1, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_MMA);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int i = 0; i < c.num_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                        report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_MMA);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if (it == 0) ET_TL(3);
                    const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(sB + s * Cfg::B_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024, SWZ_128B);
                        // MN-major: 16 K-rows = two 8-row groups of 128 bytes (SBO 1024); the
                        // next 64-column atom sits BK * 128 bytes further (LBO).
#pragma unroll
                        for (int h = 0; h < Cfg::N_HALVES; ++h) {
                            const uint32_t bh = b_addr + h * (Cfg::MMA_N * 128);
                            const uint64_t bd =
                                B_MN ? make_smem_desc(bh + k * 2048, BK * 128, 1024, SWZ_128B)
                                     : make_smem_desc(bh + k * 32, 16, 1024, SWZ_128B);
                            mma_f16_ss(d_tmem + h * Cfg::MMA_N, ad, bd, idesc,
                                       (i | k) != 0 ? 1u : 0u);
                        }
                    }
                    mma_commit(&empty_bar[s]);
                }
                if (ok) mma_commit(&acc_full[buf]);
                ET_TL(tile_iter == 0 ? 4 : 5);
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> staging -> global ----------------
        const int q = warp & 3;            // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;  // which of the quadrant's two warps this is
        const int et = threadIdx.x - 64;   // 0 .. EPI_THREADS - 1
        constexpr int NCHUNK = BN / 32;
        bool ok = true;  // a warp whose wait ran out keeps walking so that named barriers match
        int tile_iter = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_iter) {
            const TileCoord c = decode(t);
            const int buf = PERSIST ? (tile_iter & 1) : 0;
            const uint32_t use_ph = PERSIST ? ((tile_iter >> 1) & 1) : (tile_iter & 1);
            const int grp = B_MN ? c.z : 0;
            const __half* bias = g.bias ? g.bias + static_cast<size_t>(grp) * N : nullptr;
            float* tb = s_bias + buf * BN;
            int* tc = s_col + buf * BN;
            // Stage this tile's bias (and output column ids) in shared memory while its main
            // loop is still running: read per chunk from global they cost an L2 round trip.
            for (int i = et; i < BN; i += EPI_THREADS) {
                const int n = c.n0 + i;
                int feat = n;
                if (col_map != nullptr && n < N) feat = __ldg(col_map + n);
                tc[i] = feat;
                tb[i] = (bias != nullptr && n < N && g.out_mode != OUT_PARTIAL_F32)
                            ? __half2float(__ldg(bias + feat))
                            : 0.f;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            if (tile_iter == 0) pdl_wait();  // outputs may still be read by the previous kernel
            if (ok) {
                ok = mbar_wait_bounded(&acc_full[buf], use_ph, abort_flag);
                if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_EPILOGUE);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;
            tc_fence_after_sync();
            if (threadIdx.x == 64) ET_TL(tile_iter == 0 ? 7 : 8);
            // the TMA stores of this warp's previous tile must have read the staging tiles
            if (tile_iter > 0) {
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
            }

            const int row = c.m0 + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
            // This warp's share of the tile's 32-column chunks: for the fp16 tile store whole
            // 64-column groups alternate between the quadrant's two warps, otherwise chunks do.
            const bool by_group = EPI != 0 || g.out_mode == OUT_TILE_F16;
            int my_chunks[NCHUNK];
            int n_my = 0;
#pragma unroll
            for (int ch = 0; ch < NCHUNK; ++ch) {
                int owner = by_group ? ((ch >> 1) & 1) : (ch & 1);
                if (by_group && BN == 64) owner = 0;
                if (owner == half && c.n0 + ch * 32 < N) my_chunks[n_my++] = ch;
            }

            auto finish_chunk = [&](int ch, const uint32_t (&r)[32]) {
                if (EPI != 0) {
                    uint8_t* tile = sStage + (q * (BN / 64) + (ch >> 1)) * 4096;
                    stage_f16_chunk<EPI - 1>(r, tb + ch * 32, tile + lane * 128, ch & 1, lane);
                    if ((ch & 1) || c.n0 + ch * 32 + 32 >= N) {  // the 64-column group is complete
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && c.m0 + q * 32 < M)
                            tma_store_2d(&tmY, tile, c.n0 + (ch >> 1) * 64, c.m0 + q * 32);
                    }
                    return;
                }
                if (g.out_mode == OUT_TILE_F16) {
                    uint8_t* tile = sStage + (q * (BN / 64) + (ch >> 1)) * 4096;
                    uint8_t* srow = tile + lane * 128;
                    const float* b32 = tb + ch * 32;
                    if (g.act == ET_ACT_GELU)
                        stage_f16_chunk<ET_ACT_GELU>(r, b32, srow, ch & 1, lane);
                    else if (g.act == ET_ACT_RELU)
                        stage_f16_chunk<ET_ACT_RELU>(r, b32, srow, ch & 1, lane);
                    else
                        stage_f16_chunk<ET_ACT_NONE>(r, b32, srow, ch & 1, lane);
                    if ((ch & 1) || c.n0 + ch * 32 + 32 >= N) {  // the 64-column group is complete
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && c.m0 + q * 32 < M)
                            tma_store_2d(&tmY, tile, c.n0 + (ch >> 1) * 64, c.m0 + q * 32);
                    }
                } else if (g.out_mode == OUT_PARTIAL_F32) {
                    uint8_t* tile = sStage + (q * NCHUNK + ch) * 4096;
                    uint8_t* srow = tile + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        *reinterpret_cast<uint4*>(srow + ((j ^ (lane & 7)) * 16)) = v;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && c.m0 + q * 32 < M)
                        tma_store_3d(&tmY, tile, c.n0 + ch * 32, c.m0 + q * 32, c.z);
                } else if (row < M) {
                    // index-list / grouped-row epilogues: direct stores (small problems only)
                    __half* Y = static_cast<__half*>(g.Y);
                    size_t out_row = static_cast<size_t>(row);
                    if (g.grp_rows > 0)
                        out_row = static_cast<size_t>(row / g.grp_rows) * g.grp_stride +
                                  static_cast<size_t>(grp) * g.grp_rows + row % g.grp_rows;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = c.n0 + ch * 32 + j;
                        if (n < N) {
                            const float v = apply_act(__uint_as_float(r[j]) + tb[ch * 32 + j], g.act);
                            const int col = (col_map != nullptr && !g.scatter) ? n : tc[ch * 32 + j];
                            Y[out_row * g.ldy + col] = __float2half_rn(v);
                        }
                    }
                }
            };

            // software pipeline: the load of the next chunk is in flight while this one is
            // converted and staged
            uint32_t ra[32], rb[32];
            if (c.num_kb == 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) ra[j] = 0u;
                for (int i = 0; i < n_my; ++i) finish_chunk(my_chunks[i], ra);
            } else if (n_my > 0) {
                tmem_ld32(lane_addr + my_chunks[0] * 32, ra);
#pragma unroll 1
                for (int i = 0; i < n_my; i += 2) {
                    tmem_ld_wait_regs(ra);
#ifdef ET_TIMELINE
                    const long long tl_a = clock64();
#endif
                    if (i + 1 < n_my) tmem_ld32(lane_addr + my_chunks[i + 1] * 32, rb);
#ifdef ET_TIMELINE
                    const long long tl_b = clock64();
#endif
                    finish_chunk(my_chunks[i], ra);
#ifdef ET_TIMELINE
                    const long long tl_c = clock64();
#endif
                    if (i + 1 < n_my) {
                        tmem_ld_wait_regs(rb);
#ifdef ET_TIMELINE
                        const long long tl_d = clock64();
#endif
                        if (i + 2 < n_my) tmem_ld32(lane_addr + my_chunks[i + 2] * 32, ra);
                        finish_chunk(my_chunks[i + 1], rb);
#ifdef ET_TIMELINE
                        const long long tl_e = clock64();
                        if (threadIdx.x == 64 && tile_iter == 0 && i == 0 && blockIdx.x < 4096) {
                            et_gemm_timeline[blockIdx.x * 16 + 12] = tl_a;
                            et_gemm_timeline[blockIdx.x * 16 + 13] = tl_b;
                            et_gemm_timeline[blockIdx.x * 16 + 14] = tl_c;
                            et_gemm_timeline[blockIdx.x * 16 + 15] = tl_d;
                            et_gemm_timeline[blockIdx.x * 16 + 6] = tl_e;
                        }
#endif
                    }
                }
            }
            // this warp no longer needs the accumulator: hand it back to the MMA thread
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&acc_empty[buf]);
                tma_store_commit();
            }
            if (threadIdx.x == 64 && tile_iter != 0) ET_TL(9);
        }
        if (lane == 0) tma_store_wait_read();
        if (threadIdx.x == 64) ET_TL(10);
    }

    pdl_wait();  // no CTA may retire before the kernels it depends on have completed
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    if (threadIdx.x == 32) ET_TL(11);
}

// Row-pruned Linear, second step.  The GEMM has left the nn kept features of every row in the
// first nn columns of the row of Y (pitch `out`); this kernel rewrites each row in place as the
// full row: kept feature i moves to column row_id[i], every other column gets act(bias[c]).
// Every warp owns a shared-memory image of one full output row, filled once with act(bias[c]):
// the pruned columns never change.  For a row it drops the kept features into the image
// (4-byte loads that are coalesced across the warp, 2-byte shared-memory stores at ascending
// positions: few bank conflicts) and then writes the image out with 16-byte stores.
// The warps of a CTA walk rows independently (no CTA-wide barrier per row).  Shared memory:
// nn * 4 + warps * out * 2 bytes.
constexpr int EXPAND_WARPS = 8;
__global__ void __launch_bounds__(32 * EXPAND_WARPS)
expand_rows_kernel(__half* __restrict__ Y, const int* __restrict__ row_id,
                   const __half* __restrict__ bias, int rows, int out, int nn, int act) {
    extern __shared__ __align__(16) uint8_t expand_smem[];
    int* sid = reinterpret_cast<int*>(expand_smem);  // [nn] kept feature ids (nn % 8 == 0)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __half* image = reinterpret_cast<__half*>(sid + nn) + static_cast<size_t>(warp) * out;
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < nn; i += 32 * EXPAND_WARPS) {
        const int id = __ldg(row_id + i);
        sid[i] = (id >= 0 && id < out) ? id : 0;  // (validated lists never take the second arm)
    }
    // the fill values, computed once per CTA (in the last warp's image), then copied
    __half* last = reinterpret_cast<__half*>(sid + nn) + static_cast<size_t>(EXPAND_WARPS - 1) * out;
    for (int c = threadIdx.x; c < out; c += 32 * EXPAND_WARPS)
        last[c] = __float2half_rn(apply_act(bias ? __half2float(__ldg(bias + c)) : 0.f, act));
    __syncthreads();
    if (warp != EXPAND_WARPS - 1)
        for (int c = lane * 8; c < out; c += 256)
            *reinterpret_cast<uint4*>(image + c) = *reinterpret_cast<const uint4*>(last + c);
    pdl_wait();  // the tables above are weights; Y comes from the GEMM
    __syncthreads();
    unsigned short* img = reinterpret_cast<unsigned short*>(image);
    for (int r = blockIdx.x * EXPAND_WARPS + warp; r < rows; r += gridDim.x * EXPAND_WARPS) {
        const size_t base = static_cast<size_t>(r) * out;
        // pairs of kept features per load; a batch of 32 loads per lane (4 KB per warp: a whole
        // row of up to 2048 kept features) is in flight before the stores that need them
        const uint32_t* Yw = reinterpret_cast<const uint32_t*>(Y) + base / 2;
        const int npair = nn >> 1;
        for (int p0 = 0; p0 < npair; p0 += 32 * 32) {
            uint32_t v[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                const int p = p0 + u * 32 + lane;
                v[u] = p < npair ? __ldcg(Yw + p) : 0u;
            }
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                const int p = p0 + u * 32 + lane;
                if (p < npair) {
                    const int2 ids = *reinterpret_cast<const int2*>(sid + 2 * p);
                    img[ids.x] = static_cast<unsigned short>(v[u] & 0xffffu);
                    img[ids.y] = static_cast<unsigned short>(v[u] >> 16);
                }
            }
        }
        __syncwarp();  // every kept feature of the row has been read before the row is overwritten
        for (int c = lane * 8; c < out; c += 256)
            *reinterpret_cast<uint4*>(Y + base + c) = *reinterpret_cast<const uint4*>(image + c);
        __syncwarp();
    }
}

// out[r, c] = act(bias[c]) for every element: the columns a row-pruned Linear never computes.
__global__ void fill_bias_kernel(__half* __restrict__ Y, const __half* __restrict__ bias, int rows,
                                 int cols, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n8 = static_cast<size_t>(rows) * cols / 8;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>((i * 8) % cols);
        float v[8];
        if (bias != nullptr) {
            const uint4 bq = __ldg(reinterpret_cast<const uint4*>(bias + c));
            const __half2* bh = reinterpret_cast<const __half2*>(&bq);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(bh[j]);
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        }
        uint4 o;
        o.x = pack_half2(apply_act(v[0], act), apply_act(v[1], act));
        o.y = pack_half2(apply_act(v[2], act), apply_act(v[3], act));
        o.z = pack_half2(apply_act(v[4], act), apply_act(v[5], act));
        o.w = pack_half2(apply_act(v[6], act), apply_act(v[7], act));
        reinterpret_cast<uint4*>(Y)[i] = o;
    }
}

// G[t, k] = X[t, col_id[k]]: the kept input features of a column-pruned Linear.
// Row-staged form: a warp copies one row of X into a shared-memory line with coalesced 16-byte
// loads (every byte of X crosses L2 -> SM once) and, while that copy is in flight, picks the kept
// columns of the row before it from its second line, eight per lane and step, and stores them as
// 16 bytes.  The column list sits in shared memory once per CTA.  blockDim = (32, warps); dynamic
// shared memory = nn_col * 4 + warps * 2 * in * 2 bytes.  in % 8 == 0, nn_col % 8 == 0.
__global__ void gather_cols_rows_kernel(const __half* __restrict__ X, const int* __restrict__ col_id,
                                        __half* __restrict__ G, int T, int in, int nn_col) {
    extern __shared__ uint4 gather_smem[];
    const int lane = threadIdx.x, warp = threadIdx.y;
    const int ngroup = nn_col >> 3, npiece = in >> 3;
    int* ids = reinterpret_cast<int*>(gather_smem);
    uint4* lines = gather_smem + ((nn_col + 3) >> 2) + static_cast<size_t>(warp) * 2 * npiece;
    for (int i = warp * 32 + lane; i < nn_col; i += 32 * blockDim.y) ids[i] = __ldg(col_id + i);
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();
    const int stride = gridDim.x * blockDim.y;
    int t = blockIdx.x * blockDim.y + warp;
    auto fetch = [&](int row, int buf) {  // 16-byte pieces of the row into registers' worth of copies
        const uint4* xr = reinterpret_cast<const uint4*>(X + static_cast<size_t>(row) * in);
        uint4* line = lines + buf * npiece;
        for (int i = lane; i < npiece; i += 32) line[i] = __ldcg(xr + i);
    };
    int buf = 0;
    if (t < T) fetch(t, 0);
    for (; t < T; t += stride, buf ^= 1) {
        __syncwarp();
        if (t + stride < T) fetch(t + stride, buf ^ 1);
        const unsigned short* line_h = reinterpret_cast<const unsigned short*>(lines + buf * npiece);
        for (int j = lane; j < ngroup; j += 32) {
            const int4 c0 = *reinterpret_cast<const int4*>(ids + 8 * j);
            const int4 c1 = *reinterpret_cast<const int4*>(ids + 8 * j + 4);
            uint4 o;
            o.x = line_h[c0.x] | (static_cast<uint32_t>(line_h[c0.y]) << 16);
            o.y = line_h[c0.z] | (static_cast<uint32_t>(line_h[c0.w]) << 16);
            o.z = line_h[c1.x] | (static_cast<uint32_t>(line_h[c1.y]) << 16);
            o.w = line_h[c1.z] | (static_cast<uint32_t>(line_h[c1.w]) << 16);
            *reinterpret_cast<uint4*>(G + static_cast<size_t>(t) * nn_col + 8 * j) = o;
        }
    }
}

// Direct form for rows too long for a shared-memory line: a thread owns eight consecutive kept
// columns (their indices stay in registers) and walks rows: eight independent 2-byte loads and
// one 16-byte store per row.  blockDim = (gx, gy): gx threads across the column groups, gy rows
// per CTA and pass.  nn_col % 8 == 0.
__global__ void gather_cols_kernel(const __half* __restrict__ X, const int* __restrict__ col_id,
                                   __half* __restrict__ G, int T, int in, int nn_col) {
    const int ngroup = nn_col >> 3;
    const unsigned short* Xs = reinterpret_cast<const unsigned short*>(X);
    pdl_launch_dependents();
    for (int j = threadIdx.x; j < ngroup; j += blockDim.x) {
        int id[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) id[k] = __ldg(col_id + 8 * j + k);  // weights: before the wait
        pdl_wait();  // (returns at once after the first time)
        for (int t = blockIdx.x * blockDim.y + threadIdx.y; t < T; t += gridDim.x * blockDim.y) {
            const unsigned short* xr = Xs + static_cast<size_t>(t) * in;
            unsigned short h[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) h[k] = __ldcg(xr + id[k]);
            uint4 o;
            o.x = h[0] | (static_cast<uint32_t>(h[1]) << 16);
            o.y = h[2] | (static_cast<uint32_t>(h[3]) << 16);
            o.z = h[4] | (static_cast<uint32_t>(h[5]) << 16);
            o.w = h[6] | (static_cast<uint32_t>(h[7]) << 16);
            *reinterpret_cast<uint4*>(G + static_cast<size_t>(t) * nn_col + 8 * j) = o;
        }
    }
    pdl_wait();  // no CTA retires before the kernels it depends on have completed
}

int g_max_ctas = 0;  // test hook: cap on the persistent grid (0 = one CTA per SM)

template <int BN, int STAGES, bool PERSIST, bool B_MN, int EPI>
int launch_cfg_epi(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
                   GemmArgs args, int zdim, cudaStream_t stream) {
    using Cfg = GemmCfg<BN, STAGES, PERSIST>;
    auto kern = gemm_f16_kernel<BN, STAGES, PERSIST, B_MN, EPI>;
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::SMEM_BYTES) != cudaSuccess)
            return ET_ERR_CUDA;
        attr_set[dev] = true;
    }
    args.nz = zdim;
    const long tiles = static_cast<long>((args.N + BN - 1) / BN) * ((args.M + BM - 1) / BM) * zdim;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long cap = (PERSIST && g_max_ctas > 0 && g_max_ctas < sms) ? g_max_ctas : sms;
    dim3 grid(static_cast<unsigned>((PERSIST && tiles > cap) ? cap : tiles));
    return launch_kernel(kern, grid, dim3(GEMM_THREADS), Cfg::SMEM_BYTES, stream, tmA, tmB, tmY,
                         args) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

// Picks the epilogue specialisation: the fp16 tile store of a K-major product gets its
// activation compiled in; everything else uses the run-time form.
template <int BN, int STAGES, bool PERSIST, bool B_MN>
int launch_cfg(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
               const GemmArgs& args, int zdim, cudaStream_t stream) {
    if (!B_MN && args.out_mode == OUT_TILE_F16) {
        if (args.act == ET_ACT_GELU)
            return launch_cfg_epi<BN, STAGES, PERSIST, false, 1 + ET_ACT_GELU>(tmA, tmB, tmY, args, zdim, stream);
        if (args.act == ET_ACT_RELU)
            return launch_cfg_epi<BN, STAGES, PERSIST, false, 1 + ET_ACT_RELU>(tmA, tmB, tmY, args, zdim, stream);
        return launch_cfg_epi<BN, STAGES, PERSIST, false, 1 + ET_ACT_NONE>(tmA, tmB, tmY, args, zdim, stream);
    }
    return launch_cfg_epi<BN, STAGES, PERSIST, B_MN, 0>(tmA, tmB, tmY, args, zdim, stream);
}

int g_force_bn = 0;       // test hook: 0 = automatic, else 64 / 128 / 192 / 256 / 384
int g_force_persist = -1;  // test hook: -1 = automatic, 0 = single-tile CTAs, 1 = persistent

struct TilePlan {
    int bn;
    bool persist;
};

// Single-tile CTAs (two per SM) win while every tile is resident at once; beyond that the
// persistent form overlaps each tile's epilogue with the next tile's main loop.
TilePlan pick_plan(int M, int N, int K, int zdim) {
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long mt = (M + BM - 1) / BM;
    auto tiles = [&](int bn) { return mt * ((N + bn - 1) / bn) * zdim; };
    TilePlan p;
    // One 128 x 384 tile per CTA (two 192-column products per K step, 3 x 64 KB stages) covers
    // 2048 x 3072 in one round of 128 CTAs.  Measured on B200 for FFN1 (2048 x 768 -> 3072, GELU):
    // 13.6 us against 13.0 for two rounds of persistent 128 x 192 tiles - the 384-column GELU
    // epilogue is exposed after the single round - so only the test hook selects it.
    if (g_force_bn == 384) {
        p.bn = 384;
        p.persist = false;
        return p;
    }
    if (g_force_bn == 64 || g_force_bn == 128 || g_force_bn == 192 || g_force_bn == 256) {
        p.bn = g_force_bn;
        p.persist = g_force_persist >= 0 ? g_force_persist != 0 : tiles(p.bn) > (p.bn == 256 ? sms : 2 * sms);
        return p;
    }
    // Measured on B200 (K = 768 .. 8192): up to one tile per SM the one-CTA-per-SM form wins
    // (deeper ring, no register cap); up to two tiles per SM two co-resident single-tile CTAs
    // win; beyond that persistent CTAs overlap every epilogue with the next main loop; very
    // long runs prefer the widest tile (least operand traffic per FLOP).
    if (tiles(128) <= sms) {
        p.persist = true;
        p.bn = 128;
    } else if (tiles(128) <= 2L * sms && K <= 1024) {
        // (with a long K the two co-resident CTAs only share the SM's operand bandwidth)
        p.persist = false;
        p.bn = 128;
    } else if (tiles(256) >= 4L * sms) {
        p.persist = false;
        p.bn = 256;
    } else {
        // a few rounds of tiles per CTA: the width whose rounds x time per K block is least,
        // a K block costing the larger of its tensor time (2 * bn cycles) and its operand
        // bytes at the 75 B/clk an SM gets from L2 when all SMs pull
        p.persist = true;
        long best = -1;
        for (int bn : {128, 192, 256}) {
            const long rounds = (tiles(bn) + sms - 1) / sms;
            const long tensor = 2L * bn, bytes = (128L + bn) * 128 / 75;
            const long cost = rounds * (tensor > bytes ? tensor : bytes);
            if (best < 0 || cost < best) {
                best = cost;
                p.bn = bn;
            }
        }
    }
    if (g_force_persist >= 0) p.persist = g_force_persist != 0;
    return p;
}

long plan_tiles(int M, int N, int bn) {
    return static_cast<long>((M + BM - 1) / BM) * ((N + bn - 1) / bn);
}

int g_force_pair = -1;  // test hook: -1 = automatic, 0 = never, 128 / 256 = always that width

// Width of the CTA-pair tile to use for a plain [M, K] x [N, K]^T product, or 0 for the
// single-CTA kernels.
int pick_pair(int M, int N, int K) {
    if (g_force_pair == 0) return 0;
    if (g_force_pair == 128 || g_force_pair == 256) return g_force_pair;
    if (M < 2 * BM) return 0;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long mt2 = (M + 2 * BM - 1) / (2 * BM);
    // Measured on B200: 256 x 256 pair tiles win once they fill the machine more than about
    // 1.6 times over (operand traffic per FLOP is what bounds those runs); 256 x 128 pair tiles
    // win for few output tiles with a long K (every CTA streams weights for a long time and
    // halving that stream pays); otherwise fill and drain dominate and the single-CTA forms win.
    if (mt2 * ((N + 255) / 256) >= (sms / 2) * 8 / 5) return 256;
    const long single = static_cast<long>((M + BM - 1) / BM) * ((N + 127) / 128);
    if (K >= 2048 && single <= sms) return 128;
    return 0;
}

int g_force_tall = -1;  // test hook: -1 = automatic, 0 = never, 128 / 192 / 256 = always that width

// Width of the 256-row single-CTA tile to use, or 0.  That form wins when it covers the
// problem in ONE round of at most one tile per SM where 128-row tiles would need several
// rounds: the weight tile is fetched once per 256 rows, so a K block costs
// max(4 * bn, (256 + bn) * 128 B / 75) cycles for twice the rows.
int pick_tall(int M, int N, int K) {
    (void)K;
    if (g_force_tall == 0) return 0;
    if (g_force_tall == 128 || g_force_tall == 192 || g_force_tall == 256) return g_force_tall;
    // Measured on B200 (BERT-base / BERT-large FFN shapes, 2048..8192 tokens): never faster than
    // the persistent 128-row tiles or the CTA pairs - the epilogue of both accumulators is
    // exposed after the single round - so this form only runs when the test hook asks for it.
    if (g_force_tall < 0) return 0;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long mt = (M + BM - 1) / BM, mt2 = (M + 2 * BM - 1) / (2 * BM);
    if (mt * ((N + 127) / 128) <= 2L * sms) return 0;  // few tiles: the 128-row forms are resident at once
    int best_bn = 0;
    long best = -1;
    for (int bn : {256, 192, 128}) {
        const long tiles = mt2 * ((N + bn - 1) / bn);
        if (tiles > sms || tiles * 10 < sms * 6L) continue;
        const long tensor = 4L * bn, bytes = (256L + bn) * 128 / 75;
        const long cost = tensor > bytes ? tensor : bytes;
        if (best < 0 || cost < best) {
            best = cost;
            best_bn = bn;
        }
    }
    return best_bn;
}

template <bool B_MN>
int dispatch(const TilePlan& p, const CUtensorMap& tmA, const CUtensorMap& tmB,
             const CUtensorMap& tmY, const GemmArgs& args, int zdim, cudaStream_t stream) {
    if (p.bn == 192 && args.out_mode == OUT_TILE_F16 && !B_MN)
        return launch_cfg<192, 4, true, false>(tmA, tmB, tmY, args, zdim, stream);
    if (p.bn == 384 && args.out_mode == OUT_TILE_F16 && !B_MN) {
        // one 128 x 384 tile per CTA; only the compiled-in epilogues exist for this width
        if (args.act == ET_ACT_GELU)
            return launch_cfg_epi<384, 3, false, false, 1 + ET_ACT_GELU>(tmA, tmB, tmY, args, zdim, stream);
        if (args.act == ET_ACT_RELU)
            return launch_cfg_epi<384, 3, false, false, 1 + ET_ACT_RELU>(tmA, tmB, tmY, args, zdim, stream);
        return launch_cfg_epi<384, 3, false, false, 1 + ET_ACT_NONE>(tmA, tmB, tmY, args, zdim, stream);
    }
    if (p.persist) {
        if (p.bn == 256 && args.out_mode != OUT_PARTIAL_F32)
            return launch_cfg<256, 3, true, B_MN>(tmA, tmB, tmY, args, zdim, stream);
        if (p.bn == 64) return launch_cfg<64, 6, true, B_MN>(tmA, tmB, tmY, args, zdim, stream);
        return launch_cfg<128, 4, true, B_MN>(tmA, tmB, tmY, args, zdim, stream);
    }
    if (p.bn == 256 && args.out_mode != OUT_PARTIAL_F32)
        return launch_cfg<256, 4, false, B_MN>(tmA, tmB, tmY, args, zdim, stream);
    if (p.bn == 64) return launch_cfg<64, 4, false, B_MN>(tmA, tmB, tmY, args, zdim, stream);
    return launch_cfg<128, 3, false, B_MN>(tmA, tmB, tmY, args, zdim, stream);
}

GemmArgs base_args(void* Y, const __half* bias, int ldy, int M, int N, int K, int act) {
    GemmArgs a;
    a.Y = Y;
    a.bias = bias;
    a.col_map = nullptr;
    a.ldy = ldy;
    a.scatter = 0;
    a.M = M;
    a.N = N;
    a.K = K;
    a.act = act;
    a.grp_rows = 0;
    a.grp_stride = 0;
    a.out_mode = OUT_TILE_F16;
    a.kb_per_split = 0;
    a.nz = 1;
    a.err_word = device_error_word();
    return a;
}

}  // namespace

void gemm_force_bn(int bn) { g_force_bn = bn; }
void gemm_force_persist(int mode) { g_force_persist = mode; }
void gemm_set_max_ctas(int n) { g_max_ctas = n; }
void gemm_force_pair(int mode) { g_force_pair = mode; }
void gemm_force_tall(int mode) { g_force_tall = mode; }

// ---- built-in gather scratch of et_linear_col_noalloc_fwd -------------------------------
// Callers that cannot allocate device memory (see the entry point) use this array instead of
// a buffer of their own.  It is part of the library image: every GPU that loads the library
// holds these 8 MiB until the process exits.
constexpr size_t kNoAllocScratchHalves = 4u * 1024u * 1024u;  // T * nn_col may not exceed this
static __device__ __align__(256) __half g_col_gather_scratch[kNoAllocScratchHalves];

// The array's name is only a host-side handle; kernels need its device address, looked up
// once per device (with that device current) and cached.
__half* col_gather_scratch_address() {
    // several host threads may make their first call on a device at once: they all look up
    // the same address, and the slot is atomic so that none reads a half-written pointer
    static std::atomic<__half*> cached[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    __half* known = cached[dev].load(std::memory_order_acquire);
    if (known != nullptr) return known;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_col_gather_scratch) != cudaSuccess || p == nullptr)
        return nullptr;
    cached[dev].store(static_cast<__half*>(p), std::memory_order_release);
    return static_cast<__half*>(p);
}

int launch_gemm_f16(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                    __half* Y, int ldy, const int* col_map, int scatter, int M, int N, int K,
                    int act, cudaStream_t stream) {
    if (!X || !W || !Y || M <= 0 || N <= 0 || K <= 0) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (!aligned16(X) || !aligned16(W) || !aligned16(Y) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    if (ldx % 8 || ldw % 8 || K % 8) return ET_ERR_SHAPE;
    if (col_map == nullptr && (N % 8 || ldy % 8)) return ET_ERR_SHAPE;
    if (!device_error_word()) return ET_ERR_NO_DEVICE;

    if (col_map == nullptr) {
        const int pair_bn = pick_pair(M, N, K);
        if (pair_bn != 0)
            return launch_gemm_pair_f16(X, ldx, W, ldw, bias, Y, ldy, M, N, K, act, pair_bn, stream);
        const int tall_bn = pick_tall(M, N, K);
        if (tall_bn != 0)
            return launch_gemm_tall_f16(X, ldx, W, ldw, bias, Y, ldy, M, N, K, act, tall_bn, stream);
    }
    // An index list that only selects the bias (compressed output: column n of Y is feature
    // col_map[n]) keeps the coalesced tile store; only a true scatter needs per-element stores.
    const bool tile_store = col_map == nullptr || (!scatter && N % 8 == 0 && ldy % 8 == 0);
    TilePlan plan = pick_plan(M, N, K, 1);
    if (plan.bn == 384 && !tile_store) plan = TilePlan{128, plan_tiles(M, N, 128) > sm_count()};
    if (plan.bn == 192 && !tile_store) plan.bn = 128;  // 192 and 384 exist for the tile store only
    const int bn = plan.bn;
    CUtensorMap tmA, tmB;
    int st;
    if ((st = encode_operand(&tmA, X, ldx, M, K, BM)) != ET_OK) return st;
    if ((st = encode_operand(&tmB, W, ldw, N, K, bn > 256 ? bn / 2 : bn)) != ET_OK) return st;
    CUtensorMap tmY = tmA;  // placeholder when the index-list epilogue is used
    if (tile_store) {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldy) * 2};
        const uint32_t box[2] = {64, 32};
        st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    GemmArgs args = base_args(Y, bias, ldy, M, N, K, act);
    args.col_map = col_map;
    args.scatter = scatter;
    args.out_mode = tile_store ? OUT_TILE_F16 : OUT_INDEXED;
    return dispatch<false>(plan, tmA, tmB, tmY, args, 1, stream);
}

// P[s][m, n] = sum over the s-th slice of K of X[m, k] W[n, k]  (fp32, no bias): split-K
// partial sums for a consumer that adds them up (the partial-sum LayerNorm).
int launch_gemm_f16_splitk(const __half* X, int ldx, const __half* W, int ldw, float* P, int M,
                           int N, int K, int splits, cudaStream_t stream) {
    if (!X || !W || !P || M <= 0 || N <= 0 || K <= 0 || splits <= 0) return ET_ERR_INVALID_ARG;
    if (!aligned16(X) || !aligned16(W) || !aligned16(P)) return ET_ERR_ALIGNMENT;
    if (ldx % 8 || ldw % 8 || K % 8 || N % 4) return ET_ERR_SHAPE;
    if (!device_error_word()) return ET_ERR_NO_DEVICE;
    const int kb_total = (K + BK - 1) / BK;
    const int kb_per = (kb_total + splits - 1) / splits;
    CUtensorMap tmA, tmB, tmY;
    int st;
    if ((st = encode_operand(&tmA, X, ldx, M, K, BM)) != ET_OK) return st;
    if ((st = encode_operand(&tmB, W, ldw, N, K, 128)) != ET_OK) return st;
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                                  static_cast<uint64_t>(splits)};
        const uint64_t strides[2] = {static_cast<uint64_t>(N) * 4,
                                     static_cast<uint64_t>(N) * 4 * static_cast<uint64_t>(M)};
        const uint32_t box[3] = {32, 32, 1};
        st = make_tensor_map_f32(&tmY, P, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    GemmArgs args = base_args(P, nullptr, N, M, N, K, ET_ACT_NONE);
    args.out_mode = OUT_PARTIAL_F32;
    args.kb_per_split = kb_per;
    TilePlan plan;
    plan.bn = 128;
    plan.persist = static_cast<long>((M + BM - 1) / BM) * ((N + 127) / 128) * splits >
                   2L * (sm_count() > 0 ? sm_count() : 148);
    if (g_force_persist >= 0) plan.persist = g_force_persist != 0;
    return dispatch<false>(plan, tmA, tmB, tmY, args, splits, stream);
}

// Y[(m / grp_rows) * groups * grp_rows + g * grp_rows + m % grp_rows, :] = X[m, :] . W[g] + bias[g]
// for W [groups][K, N] row-major (N contiguous), bias [groups][N] or null.
int launch_gemm_f16_grouped_kn(const __half* X, int ldx, const __half* W, const __half* bias,
                               __half* Y, int M, int N, int K, int groups, int grp_rows,
                               cudaStream_t stream) {
    if (!X || !W || !Y || M <= 0 || N <= 0 || K <= 0 || groups <= 0 || grp_rows <= 0)
        return ET_ERR_INVALID_ARG;
    if (!aligned16(X) || !aligned16(W) || !aligned16(Y) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    if (ldx % 8 || K % 8 || N % 8 || groups > 65535) return ET_ERR_SHAPE;
    if (!device_error_word()) return ET_ERR_NO_DEVICE;
    TilePlan plan = pick_plan(M, N, K, groups);
    if (plan.bn == 384) plan = TilePlan{128, plan_tiles(M, N, 128) * groups > sm_count()};
    if (plan.bn == 256 || plan.bn == 192) plan.bn = 128;
    const int bn = plan.bn;
    CUtensorMap tmA, tmB;
    int st;
    if ((st = encode_operand(&tmA, X, ldx, M, K, BM)) != ET_OK) return st;
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K),
                                  static_cast<uint64_t>(groups)};
        const uint64_t strides[2] = {static_cast<uint64_t>(N) * 2,
                                     static_cast<uint64_t>(N) * 2 * static_cast<uint64_t>(K)};
        const uint32_t box[3] = {64, BK, 1};
        st = make_tensor_map_f16(&tmB, W, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    GemmArgs args = base_args(Y, bias, N, M, N, K, ET_ACT_NONE);
    args.out_mode = OUT_GROUPED;
    args.grp_rows = grp_rows;
    args.grp_stride = groups * grp_rows;
    (void)bn;
    return dispatch<true>(plan, tmA, tmB, tmA, args, groups, stream);
}

}  // namespace et

using et::launch_gemm_f16;

extern "C" {

#ifdef ET_TEST_HOOKS
// Test hook: 0 = automatic tile width, else 64 / 128 / 256.
void et_debug_force_gemm_bn(int bn) { et::gemm_force_bn(bn); }
// Test hook: cap on the number of persistent CTAs (0 = one per SM).
void et_debug_set_gemm_max_ctas(int n) { et::gemm_set_max_ctas(n); }
// Test hook: -1 = automatic, 0 = never, 128 / 192 / 256 = 256-row single-CTA tiles of that width.
void et_debug_force_gemm_tall(int mode) { et::gemm_force_tall(mode); }
// Test hook: -1 = automatic, 0 = single-CTA kernels only, 128 / 256 = CTA-pair tiles of that width.
void et_debug_force_gemm_pair(int mode) { et::gemm_force_pair(mode); }
// Test hook: -1 = automatic, 0 = one tile per CTA, 1 = persistent CTAs.
void et_debug_force_gemm_persist(int mode) { et::gemm_force_persist(mode); }
#endif  // ET_TEST_HOOKS

int et_linear_dense_fwd(const et_half* X, const et_half* W, const et_half* bias, et_half* Y,
                        int T, int in, int out, int act, et_stream stream) {
    if (in % 16 || out % 16) return (in <= 0 || out <= 0) ? ET_ERR_INVALID_ARG : ET_ERR_SHAPE;
    return launch_gemm_f16(reinterpret_cast<const __half*>(X), in,
                           reinterpret_cast<const __half*>(W), in,
                           reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(Y),
                           out, nullptr, 0, T, out, in, act, static_cast<cudaStream_t>(stream));
}

int et_linear_row_fwd(const int32_t* row_id, const et_half* rows, int nn_row,
                      const et_half* bias, const et_half* X, et_half* Y, int T, int in, int out,
                      int act, et_stream stream) {
    if (!X || !Y || T <= 0 || in <= 0 || out <= 0 || nn_row < 0 || (nn_row > 0 && (!row_id || !rows)))
        return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16) return ET_ERR_SHAPE;
    if (!et::aligned16(Y) || (bias && !et::aligned16(bias))) return ET_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Kept features first, compressed, into the head of every row of Y (coalesced tile stores),
    // then one in-place pass that spreads them and fills the pruned columns.  Measured on B200
    // with half the rows kept: 2048 x 768 -> 3072 in 17 us and 12288 x 1024 -> 4096 in 95 us,
    // against 61 us and 324 us for a bias fill of Y followed by a GEMM whose epilogue scatters
    // single elements (dense GEMM: 12.4 / 82 us; three quarters pruned: 51 us for the larger
    // shape).  Consumers that accept the compressed layout (et_linear_row_compressed_fwd, what
    // the encoder layer uses) skip the second pass altogether.
    const size_t expand_bytes =
        static_cast<size_t>(nn_row) * 4 + static_cast<size_t>(et::EXPAND_WARPS) * out * 2;
    if (nn_row > 0 && nn_row % 8 == 0 && nn_row <= out && expand_bytes <= 200 * 1024) {
        int st = launch_gemm_f16(reinterpret_cast<const __half*>(X), in,
                                 reinterpret_cast<const __half*>(rows), in,
                                 reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(Y),
                                 out, row_id, 0, T, nn_row, in, act, s);
        if (st != ET_OK) return st;
        static std::atomic<int> attr_bytes[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && attr_bytes[dev] < static_cast<int>(expand_bytes)) {
            if (cudaFuncSetAttribute(et::expand_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(expand_bytes)) != cudaSuccess)
                return ET_ERR_CUDA;
            attr_bytes[dev] = static_cast<int>(expand_bytes);
        }
        const int sms = et::sm_count() > 0 ? et::sm_count() : 148;
        const int fit = static_cast<int>((220 * 1024) / (expand_bytes + 1024));
        const int per_sm = fit > 4 ? 4 : (fit < 1 ? 1 : fit);
        const int want = (T + et::EXPAND_WARPS - 1) / et::EXPAND_WARPS;
        const int blocks = want < per_sm * sms ? want : per_sm * sms;
        return et::launch_kernel(et::expand_rows_kernel, dim3(blocks), dim3(32 * et::EXPAND_WARPS),
                                 expand_bytes, s, reinterpret_cast<__half*>(Y), row_id,
                                 reinterpret_cast<const __half*>(bias), T, out, nn_row,
                                 act) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    }
    const size_t n8 = static_cast<size_t>(T) * out / 8;
    const int blocks = static_cast<int>((n8 + 255) / 256 < 4096 ? (n8 + 255) / 256 : 4096);
    if (et::launch_kernel(et::fill_bias_kernel, dim3(blocks), dim3(256), 0, s,
                          reinterpret_cast<__half*>(Y), reinterpret_cast<const __half*>(bias), T,
                          out, act) != cudaSuccess)
        return ET_ERR_CUDA;
    if (nn_row == 0) return ET_OK;
    return launch_gemm_f16(reinterpret_cast<const __half*>(X), in,
                           reinterpret_cast<const __half*>(rows), in,
                           reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(Y),
                           out, row_id, 1, T, nn_row, in, act, s);
}

int et_linear_row_compressed_fwd(const int32_t* row_id, const et_half* rows, int nn_row,
                                 const et_half* bias, const et_half* X, et_half* Yc, int T,
                                 int in, et_stream stream) {
    if (!row_id || !rows || nn_row <= 0) return ET_ERR_INVALID_ARG;
    if (in % 16) return ET_ERR_SHAPE;
    return launch_gemm_f16(reinterpret_cast<const __half*>(X), in,
                           reinterpret_cast<const __half*>(rows), in,
                           reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(Yc),
                           nn_row, row_id, 0, T, nn_row, in, ET_ACT_NONE,
                           static_cast<cudaStream_t>(stream));
}

int et_linear_col_fwd(const int32_t* col_id, const et_half* cols, int nn_col,
                      const et_half* bias, const et_half* X, et_half* Y, int T, int in, int out,
                      int act, et_half* scratch, size_t scratch_bytes, et_stream stream) {
    if (!X || !Y || !col_id || !cols || T <= 0 || in <= 0 || out <= 0 || nn_col <= 0)
        return ET_ERR_INVALID_ARG;
    if (in % 16 || out % 16 || nn_col % 8) return ET_ERR_SHAPE;
    if (!scratch || scratch_bytes < static_cast<size_t>(T) * nn_col * sizeof(et_half))
        return ET_ERR_WORKSPACE;
    if (!et::aligned16(scratch) || !et::aligned16(X)) return ET_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int sms = et::sm_count() > 0 ? et::sm_count() : 148;
    const size_t id_bytes = ((static_cast<size_t>(nn_col) + 3) / 4) * 16;
    const size_t line_pair = static_cast<size_t>(in) * 4;  // two lines of a warp
    if (id_bytes + 2 * line_pair <= 48 * 1024) {
        // the column list and at least two warps' line pairs fit: two to eight warps per CTA,
        // a grid of a few CTAs per SM whose warps walk rows
        int warps = static_cast<int>((48 * 1024 - id_bytes) / line_pair);
        warps = warps > 8 ? 8 : warps;
        const int want = (T + warps - 1) / warps;
        const int blocks = want < 4 * sms ? want : 4 * sms;
        if (et::launch_kernel(et::gather_cols_rows_kernel, dim3(blocks), dim3(32, warps),
                              id_bytes + warps * line_pair, s, reinterpret_cast<const __half*>(X), col_id,
                              reinterpret_cast<__half*>(scratch), T, in, nn_col) != cudaSuccess)
            return ET_ERR_CUDA;
    } else {
        const int ngroup = nn_col / 8;
        const int gx = ngroup >= 256 ? 256 : ((ngroup + 31) / 32) * 32;
        const int gy = 256 / gx;
        const int want = (T + gy - 1) / gy;
        const int blocks = want < 8 * sms ? want : 8 * sms;
        if (et::launch_kernel(et::gather_cols_kernel, dim3(blocks), dim3(gx, gy), 0, s,
                              reinterpret_cast<const __half*>(X), col_id,
                              reinterpret_cast<__half*>(scratch), T, in, nn_col) != cudaSuccess)
            return ET_ERR_CUDA;
    }
    return launch_gemm_f16(reinterpret_cast<const __half*>(scratch), nn_col,
                           reinterpret_cast<const __half*>(cols), nn_col,
                           reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(Y),
                           out, nullptr, 0, T, out, nn_col, act, s);
}

int et_linear_col_noalloc_fwd(const int32_t* col_id, const et_half* cols, int nn_col,
                              const et_half* bias, const et_half* X, et_half* Y, int T, int in,
                              int out, int act, et_stream stream) {
    if (nn_col <= 0 || T <= 0) return ET_ERR_INVALID_ARG;
    if (static_cast<size_t>(T) * static_cast<size_t>(nn_col) > et::kNoAllocScratchHalves)
        return ET_ERR_WORKSPACE;  // larger than the built-in scratch: use et_linear_col_fwd
    __half* scratch = et::col_gather_scratch_address();
    if (scratch == nullptr) return ET_ERR_CUDA;
    return et_linear_col_fwd(col_id, cols, nn_col, bias, X, Y, T, in, out, act,
                             reinterpret_cast<et_half*>(scratch),
                             et::kNoAllocScratchHalves * sizeof(__half), stream);
}

int et_linear_vo_fwd(const et_half* X, const et_half* Wvo_t, const et_half* bias, et_half* VO,
                     int batch, int seq, int nhead, int emdim, et_stream stream) {
    if (batch <= 0 || seq <= 0 || nhead <= 0 || emdim <= 0) return ET_ERR_INVALID_ARG;
    if (emdim % 16) return ET_ERR_SHAPE;
    return et::launch_gemm_f16_grouped_kn(
        reinterpret_cast<const __half*>(X), emdim, reinterpret_cast<const __half*>(Wvo_t),
        reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(VO), batch * seq, emdim,
        emdim, nhead, seq, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
