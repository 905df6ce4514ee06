// Dense fp16 GEMM  Y[M, N] = act(X[M, K] . W[N, K]^T + bias)  on tcgen05 tensor cores.
//
// One CTA computes a 128 x BN output tile.  Warp 0 streams 128x64 (X) and BNx64 (W)
// K-major tiles into a ring of 128-byte-swizzled shared-memory stages with TMA; one
// thread of warp 1 issues tcgen05.mma (M=128, N=BN, K=16) with the fp32 accumulator in
// tensor memory; warps 2-9 (two per tensor-memory lane quadrant) read the accumulator back
// with software-pipelined tcgen05.ld, add the bias (staged in shared memory while the main
// loop runs), apply the activation and write the tile through a swizzled staging buffer and
// TMA stores.  Rows / columns / K beyond the problem are zero-filled by TMA on the way in
// and clipped on the way out.  Every mbarrier wait is bounded.
//
// Output modes: fp16 tile store (Linear layers), index-list store (row-pruned Linear:
// scattered or compressed columns), grouped rows (per-head V.O projection), and fp32
// split-K partials (consumed by the partial-sum LayerNorm kernel).
#include "common.cuh"
#include "kernels.h"

namespace et {

namespace {

// Optional per-CTA timestamps for bring-up builds (-DET_TIMELINE); compiled out otherwise.
#ifdef ET_TIMELINE
__device__ long long et_timeline[65536];
#define ET_TL(slot)                                                                       \
    et_timeline[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (slot)] = \
        clock64()
#else
#define ET_TL(slot) ((void)0)
#endif

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int EPI_WARPS = 8;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int A_STAGE_BYTES = BM * BK * 2;

enum : int { OUT_TILE_F16 = 0, OUT_INDEXED = 1, OUT_GROUPED = 2, OUT_PARTIAL_F32 = 3 };

template <int BN, int STAGES>
struct GemmCfg {
    static constexpr int B_STAGE_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int BAR_BYTES = 256 + 8 * BN;  // barriers + staged bias (fp32) and column ids
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + align slack
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    // the epilogue's staging tiles live in the idle pipeline stages
    static_assert(STAGES * STAGE_BYTES >= 4 * (BN / 32) * 4096, "staging does not fit");
};

// blockIdx.z selects a group (B_MN: g-th weight matrix / bias, output rows interleaved: row m
// of group g lands at (m / grp_rows) * grp_stride + g * grp_rows + m % grp_rows) or a K split
// (OUT_PARTIAL_F32: K blocks [z * kb_per_split, (z + 1) * kb_per_split)).
struct GemmArgs {
    void* Y;
    const __half* bias;
    const int* col_map;
    int ldy, scatter, M, N, K, act;
    int grp_rows, grp_stride;
    int out_mode;
    int kb_per_split;
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

// B_MN == false: W is [N, K] with K contiguous (the Linear weight layout).
// B_MN == true : W is [groups][K, N] with N contiguous; its tiles are consumed in place
//                as MN-major operands (64-column atoms of 64 K-rows, 8 KB each).
template <int BN, int STAGES, int MIN_CTAS, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, MIN_CTAS)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmY, const GemmArgs g) {
    using Cfg = GemmCfg<BN, STAGES>;
    const int zidx = blockIdx.z;
    const int grp = B_MN ? zidx : 0;
    const __half* __restrict__ bias = g.bias ? g.bias + static_cast<size_t>(grp) * g.N : nullptr;
    const int* __restrict__ col_map = g.col_map;
    const int M = g.M, N = g.N;
    int* err_word = g.err_word;

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_bias = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES + 256);
    int* s_col = reinterpret_cast<int*>(s_bias + BN);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    const int m0 = blockIdx.y * BM;
    const int kb_total = (g.K + BK - 1) / BK;
    int kb_begin = 0, kb_end = kb_total;
    if (g.out_mode == OUT_PARTIAL_F32) {
        kb_begin = zidx * g.kb_per_split;
        kb_end = kb_begin + g.kb_per_split < kb_total ? kb_begin + g.kb_per_split : kb_total;
        if (kb_end < kb_begin) kb_end = kb_begin;
    }
    const int num_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        ET_TL(0);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
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
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            int issued = 0;
            auto load_b = [&](int kb, int s) {
                if (B_MN) {
#pragma unroll
                    for (int t = 0; t < BN / 64; ++t)
                        tma_load_3d(sB + s * Cfg::B_STAGE_BYTES + t * (BK * 128), &tmB, &full_bar[s],
                                    n0 + t * 64, kb * BK, grp);
                } else {
                    tma_load_2d(sB + s * Cfg::B_STAGE_BYTES, &tmB, &full_bar[s], kb * BK, n0);
                }
            };
            // Weights do not depend on the previous kernel: fill the ring with weight tiles
            // first, then wait for the producer of the activations, then fetch those.
            const int pre = num_kb < STAGES ? num_kb : STAGES;
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&full_bar[i], Cfg::STAGE_BYTES);
                load_b(kb_begin + i, i);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                tma_load_2d(sA + i * A_STAGE_BYTES, &tmA, &full_bar[i], (kb_begin + i) * BK, m0);
                ++issued;
                if (i == 0) ET_TL(2);
            }
            for (int i = pre; i < num_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_PRODUCER);
                    break;
                }
                mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
                tma_load_2d(sA + s * A_STAGE_BYTES, &tmA, &full_bar[s], (kb_begin + i) * BK, m0);
                load_b(kb_begin + i, s);
                ++issued;
            }
            ET_TL(3);
            if (*abort_flag) {
                // Let copies already in flight land before the CTA's shared memory is released.
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int i = first; i < issued; ++i)
                    for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                        if (mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(BM, BN, 0, B_MN ? 1 : 0);
            bool ok = true;
            for (int i = 0; i < num_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_MMA);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if (i == 0) ET_TL(4);
                const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
                const uint32_t b_addr = smem_u32(sB + s * Cfg::B_STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024, SWZ_128B);
                    // MN-major: 16 K-rows = two 8-row groups of 128 bytes (SBO 1024); the next
                    // 64-column atom sits BK * 128 bytes further (LBO).
                    const uint64_t bd =
                        B_MN ? make_smem_desc(b_addr + k * 2048, BK * 128, 1024, SWZ_128B)
                             : make_smem_desc(b_addr + k * 32, 16, 1024, SWZ_128B);
                    mma_f16_ss(tmem_base, ad, bd, idesc, (i | k) != 0 ? 1u : 0u);
                }
                mma_commit(&empty_bar[s]);
            }
            if (ok) mma_commit(acc_bar);
            ET_TL(5);
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> staging -> global ----------------
        const int q = warp & 3;           // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2; // which of the quadrant's two warps this is
        const int row = m0 + q * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);

        // While the main loop runs, stage this tile's bias (and output column ids) in shared
        // memory: read per chunk from global they cost a cold L2 round trip each time.
        for (int i = threadIdx.x - 64; i < BN; i += 32 * EPI_WARPS) {
            const int n = n0 + i;
            int feat = n;
            if (col_map != nullptr && n < N) feat = __ldg(col_map + n);
            s_col[i] = feat;
            s_bias[i] = (bias != nullptr && n < N && g.out_mode != OUT_PARTIAL_F32)
                            ? __half2float(__ldg(bias + feat))
                            : 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
        pdl_wait();  // output buffers may still be read by the previous kernel until here
        bool ok = true;
        if (num_kb > 0) {
            ok = mbar_wait_bounded(acc_bar, 0, abort_flag);
            if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_EPILOGUE);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
            if (threadIdx.x == 64) ET_TL(6);
            // This warp's share of the tile's 32-column chunks: for the fp16 tile store whole
            // 64-column groups alternate between the quadrant's two warps, otherwise chunks do.
            const bool by_group = g.out_mode == OUT_TILE_F16;
            constexpr int NCHUNK = BN / 32;
            int my_chunks[NCHUNK];
            int n_my = 0;
#pragma unroll
            for (int c = 0; c < NCHUNK; ++c) {
                int owner = by_group ? ((c >> 1) & 1) : (c & 1);
                if (by_group && BN == 64) owner = 0;
                if (owner == half && n0 + c * 32 < N) my_chunks[n_my++] = c;
            }

#ifdef ET_TL_SOLO
            if (warp != 2) n_my = 0;  // bring-up experiment: one epilogue warp alone
#endif
            auto finish_chunk = [&](int c, const uint32_t (&r)[32]) {
                if (g.out_mode == OUT_TILE_F16) {
                    uint8_t* tile = smem + (q * (BN / 64) + (c >> 1)) * 4096;
                    uint8_t* srow = tile + lane * 128;
                    const float* b32 = s_bias + c * 32;
                    if (g.act == ET_ACT_GELU)
                        stage_f16_chunk<ET_ACT_GELU>(r, b32, srow, c & 1, lane);
                    else if (g.act == ET_ACT_RELU)
                        stage_f16_chunk<ET_ACT_RELU>(r, b32, srow, c & 1, lane);
                    else
                        stage_f16_chunk<ET_ACT_NONE>(r, b32, srow, c & 1, lane);
                    if (threadIdx.x == 64 && c < 2) ET_TL(10 + 3 * c);
                    if ((c & 1) || n0 + c * 32 + 32 >= N) {  // the 64-column group is complete
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (threadIdx.x == 64 && c < 2) ET_TL(14);
                        if (lane == 0 && m0 + q * 32 < M)
                            tma_store_2d(&tmY, tile, n0 + (c >> 1) * 64, m0 + q * 32);
                        if (threadIdx.x == 64 && c < 2) ET_TL(15);
                    }
                } else if (g.out_mode == OUT_PARTIAL_F32) {
                    uint8_t* tile = smem + (q * NCHUNK + c) * 4096;
                    uint8_t* srow = tile + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        *reinterpret_cast<uint4*>(srow + ((j ^ (lane & 7)) * 16)) = v;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && m0 + q * 32 < M)
                        tma_store_3d(&tmY, tile, n0 + c * 32, m0 + q * 32, zidx);
                } else if (row < M) {
                    // index-list / grouped-row epilogues: direct stores (small problems only)
                    __half* Y = static_cast<__half*>(g.Y);
                    size_t out_row = static_cast<size_t>(row);
                    if (g.grp_rows > 0)
                        out_row = static_cast<size_t>(row / g.grp_rows) * g.grp_stride +
                                  static_cast<size_t>(grp) * g.grp_rows + row % g.grp_rows;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = n0 + c * 32 + j;
                        if (n < N) {
                            const float v =
                                apply_act(__uint_as_float(r[j]) + s_bias[c * 32 + j], g.act);
                            const int col = (col_map != nullptr && !g.scatter) ? n : s_col[c * 32 + j];
                            Y[out_row * g.ldy + col] = __float2half_rn(v);
                        }
                    }
                }
            };

            // software pipeline: the load of the next chunk is in flight while this one is
            // converted and staged
            uint32_t ra[32], rb[32];
            if (num_kb == 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) ra[j] = 0u;
                for (int i = 0; i < n_my; ++i) finish_chunk(my_chunks[i], ra);
            } else if (n_my > 0) {
                tmem_ld32(lane_addr + my_chunks[0] * 32, ra);
#pragma unroll 1
                for (int i = 0; i < n_my; i += 2) {
                    tmem_ld_wait_regs(ra);
                    if (threadIdx.x == 64 && i == 0) ET_TL(9);
                    if (i + 1 < n_my) tmem_ld32(lane_addr + my_chunks[i + 1] * 32, rb);
                    finish_chunk(my_chunks[i], ra);
                    if (i + 1 < n_my) {
                        tmem_ld_wait_regs(rb);
                        if (threadIdx.x == 64 && i == 0) ET_TL(12);
                        if (i + 2 < n_my) tmem_ld32(lane_addr + my_chunks[i + 2] * 32, ra);
                        finish_chunk(my_chunks[i + 1], rb);
                    }
                }
            }
            if (g.out_mode == OUT_TILE_F16 || g.out_mode == OUT_PARTIAL_F32) {
                if (lane == 0) {
                    tma_store_commit();
                    tma_store_wait_read();
                }
            }
        }
    }

    if (threadIdx.x == 64) ET_TL(7);
    pdl_wait();  // no CTA may retire before the kernels it depends on have completed
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) ET_TL(8);
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
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
__global__ void gather_cols_kernel(const __half* __restrict__ X, const int* __restrict__ col_id,
                                   __half* __restrict__ G, int T, int in, int nn_col) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = static_cast<size_t>(T) * nn_col;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = i / nn_col;
        const int k = static_cast<int>(i - t * nn_col);
        G[i] = X[t * in + __ldg(col_id + k)];
    }
}

template <int BN, int STAGES, int MIN_CTAS, bool B_MN>
int launch_cfg(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
               const GemmArgs& args, int zdim, cudaStream_t stream) {
    using Cfg = GemmCfg<BN, STAGES>;
    auto kern = gemm_f16_kernel<BN, STAGES, MIN_CTAS, B_MN>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::SMEM_BYTES) != cudaSuccess)
            return ET_ERR_CUDA;
        attr_set[dev] = true;
    }
    dim3 grid((args.N + BN - 1) / BN, (args.M + BM - 1) / BM, zdim);
    return launch_kernel(kern, grid, dim3(GEMM_THREADS), Cfg::SMEM_BYTES, stream, tmA, tmB, tmY,
                         args) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

int g_force_bn = 0;

int pick_bn(int M, int N, int groups = 1) {
    if (g_force_bn == 64 || g_force_bn == 128 || g_force_bn == 256) return g_force_bn;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const int mt = (M + BM - 1) / BM;
    int best_bn = 128;
    long best_cost = -1;
    const int cands[3] = {256, 128, 64};
    for (int bn : cands) {
        const long tiles = static_cast<long>(mt) * ((N + bn - 1) / bn) * groups;
        const long waves = (tiles + sms - 1) / sms;
        const long cost = waves * (bn + 48);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_bn = bn;
        }
    }
    return best_bn;
}

int encode_operand(CUtensorMap* tm, const __half* p, int ld, int rows, int K, int box_rows) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ld) * 2};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(box_rows)};
    return make_tensor_map_f16(tm, p, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
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
    a.err_word = device_error_word();
    return a;
}

}  // namespace

void gemm_force_bn(int bn) { g_force_bn = bn; }

// ---- built-in gather scratch of et_linear_col_noalloc_fwd -------------------------------
// Callers that cannot allocate device memory (see the entry point) use this array instead of
// a buffer of their own.  It is part of the library image: every GPU that loads the library
// holds these 8 MiB until the process exits.
constexpr size_t kNoAllocScratchHalves = 4u * 1024u * 1024u;  // T * nn_col may not exceed this
static __device__ __align__(256) __half g_col_gather_scratch[kNoAllocScratchHalves];

// The array's name is only a host-side handle; kernels need its device address, looked up
// once per device (with that device current) and cached.
__half* col_gather_scratch_address() {
    static __half* cached[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] != nullptr) return cached[dev];
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_col_gather_scratch) != cudaSuccess || p == nullptr)
        return nullptr;
    cached[dev] = static_cast<__half*>(p);
    return cached[dev];
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

    const int bn = pick_bn(M, N);
    CUtensorMap tmA, tmB;
    int st;
    if ((st = encode_operand(&tmA, X, ldx, M, K, BM)) != ET_OK) return st;
    if ((st = encode_operand(&tmB, W, ldw, N, K, bn)) != ET_OK) return st;
    CUtensorMap tmY = tmA;  // placeholder when the index-list epilogue is used
    if (col_map == nullptr) {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldy) * 2};
        const uint32_t box[2] = {64, 32};
        st = make_tensor_map_f16(&tmY, Y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != ET_OK) return st;
    }
    GemmArgs args = base_args(Y, bias, ldy, M, N, K, act);
    args.col_map = col_map;
    args.scatter = scatter;
    args.out_mode = col_map == nullptr ? OUT_TILE_F16 : OUT_INDEXED;
    switch (bn) {
        case 256: return launch_cfg<256, 4, 1, false>(tmA, tmB, tmY, args, 1, stream);
        case 64: return launch_cfg<64, 4, 2, false>(tmA, tmB, tmY, args, 1, stream);
        default: return launch_cfg<128, 3, 2, false>(tmA, tmB, tmY, args, 1, stream);
    }
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
    return launch_cfg<128, 3, 2, false>(tmA, tmB, tmY, args, splits, stream);
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
    const int bn = pick_bn(M, N, groups) == 64 ? 64 : 128;
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
    if (bn == 64) return launch_cfg<64, 4, 2, true>(tmA, tmB, tmA, args, groups, stream);
    return launch_cfg<128, 3, 2, true>(tmA, tmB, tmA, args, groups, stream);
}

}  // namespace et

using et::launch_gemm_f16;

extern "C" {

// Test hook: 0 = automatic tile width, else 64 / 128 / 256.
void et_debug_force_gemm_bn(int bn) { et::gemm_force_bn(bn); }

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
    if (!et::aligned16(scratch)) return ET_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t total = static_cast<size_t>(T) * nn_col;
    const int blocks = static_cast<int>((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
    if (et::launch_kernel(et::gather_cols_kernel, dim3(blocks), dim3(256), 0, s,
                          reinterpret_cast<const __half*>(X), col_id,
                          reinterpret_cast<__half*>(scratch), T, in, nn_col) != cudaSuccess)
        return ET_ERR_CUDA;
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
