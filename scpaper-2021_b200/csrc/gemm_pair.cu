// Dense fp16 GEMM  Y[M, N] = act(X[M, K] . W[N, K]^T + bias)  on CTA pairs.
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256 x BN output tile with
// tcgen05.mma.cta_group::2: each CTA loads only ITS 128 rows of X and ITS BN/2 rows of W, the
// tensor cores of both SMs read both halves of W, and each CTA keeps its 128 x BN half of the
// accumulator in its own tensor memory.  Per FLOP a CTA pulls half the weight bytes of a
// single-CTA 128 x BN tile out of L2: 64 B/clk/SM at full tensor rate for BN = 256, which the
// L2 sustains with all SMs pulling, where the single-CTA tiles (96..128 B/clk/SM) do not.
// Every CTA fetches its own operands (no cluster-wide fan-out of loads); their completion is
// signalled straight on the leader's barrier.
//
// Roles per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (leader CTA only; in both CTAs it
// owns the tensor-memory allocation), warps 2-9 = epilogue of the CTA's own 128 rows (same
// staging + TMA-store epilogue as the single-CTA kernel).  Persistent over a static list of
// pair tiles, two accumulators, every wait bounded.
#include "common.cuh"
#include "gemm_common.cuh"
#include "kernels.h"

namespace et {

// Bring-up aid: with -DET_TIMELINE every CTA records clock64() at a few points of its life.
#ifdef ET_TIMELINE
__device__ long long et_pair_timeline[4096 * 16];
#define ET_TL(slot) \
    do { if (blockIdx.x < 4096) et_pair_timeline[blockIdx.x * 16 + (slot)] = clock64(); } while (0)
#else
#define ET_TL(slot) ((void)0)
#endif

namespace {

using namespace gemm;

// PERSIST: one CTA pair per SM pair walks several tiles with two accumulators, so that a tile's
// epilogue overlaps the next tile's main loop.  !PERSIST: one tile per CTA pair, one
// accumulator, the staging tiles reuse the then idle ring; small enough (shared memory and
// tensor memory) for two CTAs per SM, so that the next kernel's CTAs can start (programmatic
// dependent launch) while this kernel's epilogues drain.
// PARTIAL (single-tile form only): the tile index carries a K split; the epilogue writes
// the fp32 partial sums of its K slice (no bias) through fp32 staging tiles in the idle ring.
template <int BN, int STAGES, bool PERSIST, bool PARTIAL = false>
struct PairCfg {
    static constexpr int B_HALF_BYTES = (BN / 2) * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_HALF_BYTES;  // per CTA
    static constexpr int STAGING_NEED = BN * 256;  // 4 quadrants x BN/64 groups x 4 KB
    static constexpr int STAGING_BYTES = (PERSIST && !PARTIAL) ? STAGING_NEED : 0;
    static constexpr int MISC_BYTES = 256 + 2 * 4 * BN;  // barriers + 2 x bias fp32
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + MISC_BYTES + 1024;
    static constexpr int NACC = PERSIST ? 2 : 1;
    static constexpr int TMEM_COLS = NACC * BN;
    static constexpr int MIN_CTAS = (PERSIST || PARTIAL) ? 1 : 2;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget exceeded");
    static_assert(!PERSIST || SMEM_BYTES > 114 * 1024, "persistent form: one CTA per SM is assumed");
    static_assert(!PARTIAL || !PERSIST, "partial sums exist in the single-tile form only");
    static_assert(PERSIST || PARTIAL || SMEM_BYTES <= 113 * 1024, "single-tile form: two CTAs per SM");
    static_assert(PERSIST || STAGES * STAGE_BYTES >= (PARTIAL ? 2 : 1) * STAGING_NEED,
                  "staging does not fit the ring");
    static_assert(TMEM_COLS * MIN_CTAS <= 512 && STAGES <= 8, "budget exceeded");
};

struct PairTile {
    int n0, m0;
};

// ACT: the activation, compiled in (run-time branches around the staging code cost a factor
// of three in the epilogue).
template <int BN, int STAGES, bool PERSIST, bool PARTIAL, int ACT>
__global__ void __cluster_dims__(2, 1, 1)
__launch_bounds__(GEMM_THREADS, (PairCfg<BN, STAGES, PERSIST, PARTIAL>::MIN_CTAS))
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmY, const GemmArgs g) {
    using Cfg = PairCfg<BN, STAGES, PERSIST, PARTIAL>;
    const int M = g.M, N = g.N;
    int* err_word = g.err_word;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    // single-tile form: every product of the tile has completed before the epilogue runs
    uint8_t* sStage = PERSIST ? smem + STAGES * Cfg::STAGE_BYTES : smem;
    uint8_t* misc = smem + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);  // used in the leader
    uint64_t* empty_bar = full_bar + 8;
    uint64_t* acc_full = empty_bar + 8;   // [2]
    uint64_t* acc_empty = acc_full + 2;   // [2], used in the leader: both CTAs' epilogue warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_bias = reinterpret_cast<float*>(misc + 256);  // [2][BN]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles_n = (N + BN - 1) / BN;
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
    const int tiles_mn = tiles_n * tiles_m;
    const int total_tiles = tiles_mn * (PARTIAL ? g.nz : 1);
    const int kb_total = (g.K + BK - 1) / BK;
    // K blocks of this CTA's tile(s): everything, or (PARTIAL: one tile per pair) the split's slice
    int kb_begin = 0, num_kb = kb_total;
    const int split = PARTIAL ? pair / tiles_mn : 0;
    if (PARTIAL) {
        kb_begin = split * g.kb_per_split;
        int kb_end = kb_begin + g.kb_per_split < kb_total ? kb_begin + g.kb_per_split : kb_total;
        if (kb_end < kb_begin) kb_end = kb_begin;
        num_kb = kb_end - kb_begin;
    }

    auto decode = [&](int t) {
        PairTile c;
        const int tt = PARTIAL ? t % tiles_mn : t;
        c.n0 = (tt % tiles_n) * BN;
        c.m0 = (tt / tiles_n) * 2 * BM + static_cast<int>(rank) * BM;  // this CTA's rows
        return c;
    };

    if (threadIdx.x == 0) ET_TL(0);
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 2 * EPI_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) ET_TL(1);
    cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them
    tc_fence_after_sync();
    if (threadIdx.x == 0) ET_TL(2);
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (elect_one()) {
            int s = 0, issued = 0;
            uint32_t ph = 0;
            bool ok = true;
            bool first = true;
            for (int t = pair; ok && t < total_tiles; t += npairs) {
                const PairTile c = decode(t);
                const int nb0 = c.n0 + static_cast<int>(rank) * (BN / 2);  // this CTA's rows of W
                int i0 = 0;
                if (first) {
                    // weights do not depend on the previous kernel: fetch them before waiting
                    // for the producer of the activations
                    first = false;
                    const int pre = num_kb < STAGES ? num_kb : STAGES;
                    for (int i = 0; i < pre; ++i) {
                        if (rank == 0) mbar_arrive_expect_tx(&full_bar[i], 2 * Cfg::STAGE_BYTES);
                        tma_load_2d_pair(sB + i * Cfg::B_HALF_BYTES, &tmB,
                                         map_to_cta(smem_u32(&full_bar[i]), 0), (kb_begin + i) * BK,
                                         nb0);
                    }
                    ET_TL(3);
                    pdl_wait();
                    ET_TL(4);
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d_pair(sA + i * A_STAGE_BYTES, &tmA,
                                         map_to_cta(smem_u32(&full_bar[i]), 0), (kb_begin + i) * BK,
                                         c.m0);
                    issued = pre;
                    s = pre % STAGES;
                    ph = (pre / STAGES) & 1;
                    i0 = pre;
                }
                for (int i = i0; i < num_kb; ++i) {
                    if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                        report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * Cfg::STAGE_BYTES);
                    const uint32_t lb = map_to_cta(smem_u32(&full_bar[s]), 0);
                    tma_load_2d_pair(sA + s * A_STAGE_BYTES, &tmA, lb, (kb_begin + i) * BK, c.m0);
                    tma_load_2d_pair(sB + s * Cfg::B_HALF_BYTES, &tmB, lb, (kb_begin + i) * BK, nb0);
                    ++issued;
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (*abort_flag && rank == 0) {
                // Let copies in flight land before shared memory is released: both CTAs' loads
                // signal the leader's barriers, and the peer cannot leave before the leader has
                // reached the final cluster barrier, so this wait covers the peer's copies too.
                for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
                    for (uint32_t sp = 0; sp < ET_SPIN_LIMIT; ++sp)
                        if (mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA) ----------------
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, 0, 0);
            int s = 0, tile_iter = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = pair; ok && t < total_tiles; t += npairs, ++tile_iter) {
                const int buf = PERSIST ? (tile_iter & 1) : 0;
                const uint32_t use_ph = (tile_iter >> 1) & 1;
                // both CTAs' epilogues must have drained this accumulator's previous tile
                if (PERSIST && !mbar_wait_bounded(&acc_empty[buf], use_ph ^ 1, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_MMA);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int i = 0; i < num_kb; ++i) {
                    if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                        report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_MMA);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if (tile_iter == 0 && i == 0) ET_TL(5);
                    const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(sB + s * Cfg::B_HALF_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024, SWZ_128B);
                        const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024, SWZ_128B);
                        mma_f16_ss_pair(d_tmem, ad, bd, idesc, (i | k) != 0 ? 1u : 0u);
                    }
                    // the stage is free in both CTAs once these products have read it
                    const uint32_t eb = smem_u32(&empty_bar[s]);
                    mma_commit_pair(eb);
                    mma_commit_pair(map_to_cta(eb, 1));
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) {
                    const uint32_t af = smem_u32(&acc_full[buf]);
                    mma_commit_pair(af);
                    mma_commit_pair(map_to_cta(af, 1));
                    ET_TL(6);
                }
            }
        }
    } else {
        // ---------------- epilogue of this CTA's 128 rows ----------------
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int et = threadIdx.x - 64;
        constexpr int NCHUNK = BN / 32;
        bool ok = true;
        int tile_iter = 0;
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(&acc_empty[0]), 0);
        for (int t = pair; t < total_tiles; t += npairs, ++tile_iter) {
            const PairTile c = decode(t);
            const int buf = PERSIST ? (tile_iter & 1) : 0;
            const uint32_t use_ph = PERSIST ? ((tile_iter >> 1) & 1) : (tile_iter & 1);
            float* tb = s_bias + buf * BN;
            for (int i = et; i < BN; i += EPI_THREADS) {
                const int n = c.n0 + i;
                tb[i] = (!PARTIAL && g.bias != nullptr && n < N) ? __half2float(__ldg(g.bias + n)) : 0.f;
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
            if (threadIdx.x == 64) ET_TL(7);
            if (tile_iter > 0) {
                if (lane == 0) tma_store_wait_read();  // staging tiles of the previous tile
                __syncwarp();
            }

            const uint32_t lane_addr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
            int my_chunks[NCHUNK];
            int n_my = 0;
#pragma unroll
            for (int ch = 0; ch < NCHUNK; ++ch)
                if (((ch >> 1) & 1) == half && c.n0 + ch * 32 < N) my_chunks[n_my++] = ch;

            auto finish_chunk = [&](int ch, const uint32_t (&r)[32]) {
                if (PARTIAL) {
                    // 32 rows x 32 fp32 columns: one swizzled 4 KB staging tile, one TMA store
                    uint8_t* tile = sStage + (q * NCHUNK + ch) * 4096;
                    uint8_t* srow = tile + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(srow + ((j ^ (lane & 7)) * 16)) =
                            make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && c.m0 + q * 32 < M)
                        tma_store_3d(&tmY, tile, c.n0 + ch * 32, c.m0 + q * 32, split);
                    return;
                }
                uint8_t* tile = sStage + (q * (BN / 64) + (ch >> 1)) * 4096;
                uint8_t* srow = tile + lane * 128;
                const float* b32 = tb + ch * 32;
                stage_f16_chunk<ACT>(r, b32, srow, ch & 1, lane);
                if ((ch & 1) || c.n0 + ch * 32 + 32 >= N) {  // the 64-column group is complete
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && c.m0 + q * 32 < M)
                        tma_store_2d(&tmY, tile, c.n0 + (ch >> 1) * 64, c.m0 + q * 32);
                }
            };

            uint32_t ra[32], rb[32];
            if (num_kb == 0) {  // an empty K slice: no product ran, the partial sum is zero
#pragma unroll
                for (int j = 0; j < 32; ++j) ra[j] = 0u;
                for (int i = 0; i < n_my; ++i) finish_chunk(my_chunks[i], ra);
            } else if (n_my > 0) {
                tmem_ld32(lane_addr + my_chunks[0] * 32, ra);
#pragma unroll 1
                for (int i = 0; i < n_my; i += 2) {
                    tmem_ld_wait_regs(ra);
                    if (i + 1 < n_my) tmem_ld32(lane_addr + my_chunks[i + 1] * 32, rb);
                    finish_chunk(my_chunks[i], ra);
                    if (i + 1 < n_my) {
                        tmem_ld_wait_regs(rb);
                        if (i + 2 < n_my) tmem_ld32(lane_addr + my_chunks[i + 2] * 32, ra);
                        finish_chunk(my_chunks[i + 1], rb);
                    }
                }
            }
            // this warp no longer needs the accumulator: tell the leader's MMA thread
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PERSIST) {
                    if (rank == 0)
                        mbar_arrive(&acc_empty[buf]);
                    else
                        mbar_arrive_cluster(leader_acc_empty + buf * 8);
                }
                tma_store_commit();
            }
        }
        if (threadIdx.x == 64) ET_TL(8);
        if (lane == 0) tma_store_wait_read();
        if (threadIdx.x == 64) ET_TL(9);
    }

    pdl_wait();  // no CTA may retire before the kernels it depends on have completed
    tc_fence_before_sync();
    __syncthreads();
    // neither CTA may leave while the other can still read its shared memory (operand halves)
    // or arrive on its barriers
    if (threadIdx.x == 0) ET_TL(10);
    cluster_sync_all();
    if (threadIdx.x == 0) ET_TL(11);
    if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    if (threadIdx.x == 32) ET_TL(12);
}

template <int BN, int STAGES, bool PERSIST, bool PARTIAL, int ACT>
int launch_pair_act(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
                    const GemmArgs& args, cudaStream_t stream) {
    using Cfg = PairCfg<BN, STAGES, PERSIST, PARTIAL>;
    auto kern = gemm_pair_kernel<BN, STAGES, PERSIST, PARTIAL, ACT>;
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::SMEM_BYTES) != cudaSuccess)
            return ET_ERR_CUDA;
        attr_set[dev] = true;
    }
    const long tiles = static_cast<long>((args.N + BN - 1) / BN) *
                       ((args.M + 2 * BM - 1) / (2 * BM)) * (PARTIAL ? args.nz : 1);
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long pairs = (!PERSIST || tiles < sms / 2) ? tiles : sms / 2;
    return launch_kernel(kern, dim3(static_cast<unsigned>(2 * pairs)), dim3(GEMM_THREADS),
                         Cfg::SMEM_BYTES, stream, tmA, tmB, tmY, args) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

template <int BN, int STAGES, bool PERSIST, bool PARTIAL = false>
int launch_pair_cfg(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
                    const GemmArgs& args, cudaStream_t stream) {
    if (!PARTIAL && args.act == ET_ACT_GELU)
        return launch_pair_act<BN, STAGES, PERSIST, PARTIAL, ET_ACT_GELU>(tmA, tmB, tmY, args, stream);
    if (!PARTIAL && args.act == ET_ACT_RELU)
        return launch_pair_act<BN, STAGES, PERSIST, PARTIAL, ET_ACT_RELU>(tmA, tmB, tmY, args, stream);
    return launch_pair_act<BN, STAGES, PERSIST, PARTIAL, ET_ACT_NONE>(tmA, tmB, tmY, args, stream);
}

int g_pair_persist = -1;  // test hook: -1 = automatic, 0 = single-tile pairs, 1 = persistent

}  // namespace

void gemm_pair_force_persist(int mode) { g_pair_persist = mode; }

// bn: 128 or 256 (width of the pair tile).  Same contract as launch_gemm_f16 without an index
// list.
int launch_gemm_pair_f16(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                         __half* Y, int ldy, int M, int N, int K, int act, int bn,
                         cudaStream_t stream) {
    if (!X || !W || !Y || M <= 0 || N <= 0 || K <= 0) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (!aligned16(X) || !aligned16(W) || !aligned16(Y) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    if (ldx % 8 || ldw % 8 || K % 8 || N % 8 || ldy % 8) return ET_ERR_SHAPE;
    if (bn != 128 && bn != 256) return ET_ERR_INVALID_ARG;
    if (!device_error_word()) return ET_ERR_NO_DEVICE;
    CUtensorMap tmA, tmB, tmY;
    int st;
    if ((st = gemm::encode_operand(&tmA, X, ldx, M, K, gemm::BM)) != ET_OK) return st;
    if ((st = gemm::encode_operand(&tmB, W, ldw, N, K, bn / 2)) != ET_OK) return st;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldy) * 2};
        const uint32_t box[2] = {64, 32};
        st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    gemm::GemmArgs a;
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
    a.out_mode = gemm::OUT_TILE_F16;
    a.kb_per_split = 0;
    a.nz = 1;
    a.err_word = device_error_word();
    // Measured on B200: persistent pairs (a tile's epilogue overlaps the next tile's main loop)
    // win except for wide tiles with a very long K, where two co-resident single-tile CTAs per
    // SM do.
    const bool persist = g_pair_persist >= 0 ? g_pair_persist != 0 : !(bn == 256 && K >= 4096);
    if (bn == 256)
        return persist ? launch_pair_cfg<256, 4, true>(tmA, tmB, tmY, a, stream)
                       : launch_pair_cfg<256, 3, false>(tmA, tmB, tmY, a, stream);
    return persist ? launch_pair_cfg<128, 6, true>(tmA, tmB, tmY, a, stream)
                   : launch_pair_cfg<128, 4, false>(tmA, tmB, tmY, a, stream);
}

}  // namespace et

namespace et {

// P[s][m, n] = sum over the s-th slice of K of X[m, k] W[n, k] (fp32, no bias) on 256 x 256
// pair tiles, one tile and slice per CTA pair: for products with few output tiles and a long K,
// where splitting K is what fills the machine.
int launch_gemm_pair_splitk(const __half* X, int ldx, const __half* W, int ldw, float* P, int M,
                            int N, int K, int splits, cudaStream_t stream) {
    if (!X || !W || !P || M <= 0 || N <= 0 || K <= 0 || splits <= 0) return ET_ERR_INVALID_ARG;
    if (!aligned16(X) || !aligned16(W) || !aligned16(P)) return ET_ERR_ALIGNMENT;
    if (ldx % 8 || ldw % 8 || K % 8 || N % 8) return ET_ERR_SHAPE;
    if (!device_error_word()) return ET_ERR_NO_DEVICE;
    CUtensorMap tmA, tmB, tmY;
    int st;
    if ((st = gemm::encode_operand(&tmA, X, ldx, M, K, gemm::BM)) != ET_OK) return st;
    if ((st = gemm::encode_operand(&tmB, W, ldw, N, K, 128)) != ET_OK) return st;
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                                  static_cast<uint64_t>(splits)};
        const uint64_t strides[2] = {static_cast<uint64_t>(N) * 4,
                                     static_cast<uint64_t>(N) * 4 * static_cast<uint64_t>(M)};
        const uint32_t box[3] = {32, 32, 1};
        st = make_tensor_map_f32(&tmY, P, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    const int kb_total = (K + gemm::BK - 1) / gemm::BK;
    gemm::GemmArgs a;
    a.Y = P;
    a.bias = nullptr;
    a.col_map = nullptr;
    a.ldy = N;
    a.scatter = 0;
    a.M = M;
    a.N = N;
    a.K = K;
    a.act = ET_ACT_NONE;
    a.grp_rows = 0;
    a.grp_stride = 0;
    a.out_mode = gemm::OUT_PARTIAL_F32;
    a.kb_per_split = (kb_total + splits - 1) / splits;
    a.nz = splits;
    a.err_word = device_error_word();
    return launch_pair_cfg<256, 6, false, true>(tmA, tmB, tmY, a, stream);
}

}  // namespace et

#ifdef ET_TEST_HOOKS
extern "C" {
// Test hook: -1 = automatic, 0 = one tile per CTA pair, 1 = persistent CTA pairs.
void et_debug_force_gemm_pair_persist(int mode) { et::gemm_pair_force_persist(mode); }
}
#endif  // ET_TEST_HOOKS
