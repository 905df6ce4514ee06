// Dense fp16 GEMM  Y[M, N] = act(X[M, K] . W[N, K]^T + bias)  on 256 x BN tiles, one per CTA.
//
// A single-CTA 128 x BN tile pulls (128 + BN) * 128 bytes per K block out of L2 for 2 * BN
// tensor cycles - more than the 75 B/clk an SM gets when all SMs pull - so it runs operand
// bound.  This form stacks two 128-row blocks of X on one BN-row block of W: the weight tile is
// fetched once for both, (256 + BN) * 128 bytes per 4 * BN tensor cycles (73 B/clk for BN = 192),
// and the two products of a K step go to two accumulators in tensor memory.  It is the
// single-CTA counterpart of the CTA-pair kernel (no cross-CTA synchronisation) and pays when
// the problem has about one such tile per SM: FFN1 of BERT-base at 2048 tokens is 128 tiles of
// 256 x 192 on 148 SMs, one round instead of two.
//
// Roles as in the other GEMM kernels: warp 0 = TMA producer (one 256-row box of X, one BN-row
// box of W per K block), warp 1 = MMA issuer, warps 2-9 = epilogue (both accumulators; staging
// tiles in the then idle ring, TMA stores).  Every wait is bounded.
#include "common.cuh"
#include "gemm_common.cuh"
#include "kernels.h"

namespace et {

namespace {

using namespace gemm;

template <int BN, int STAGES>
struct TallCfg {
    static constexpr int A_BYTES = 2 * A_STAGE_BYTES;  // 256 rows x 64 columns
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGING_BYTES = 2 * BN * 256;  // both accumulators' staging tiles
    static constexpr int MISC_BYTES = 256 + 4 * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + MISC_BYTES + 1024;
    static constexpr int TMEM_COLS = 2 * BN <= 256 ? 256 : 512;
    static_assert(BN % 64 == 0 && BN <= 256, "tile width");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget exceeded");
    static_assert(SMEM_BYTES > 114 * 1024, "one CTA per SM is assumed (tensor memory is taken whole)");
    static_assert(STAGES * STAGE_BYTES >= STAGING_BYTES, "staging does not fit the ring");
};

template <int BN, int STAGES, int ACT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tall_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmY, const GemmArgs g) {
    using Cfg = TallCfg<BN, STAGES>;
    const int M = g.M, N = g.N;
    int* err_word = g.err_word;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* misc = smem + STAGES * Cfg::STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
    uint64_t* empty_bar = full_bar + 8;
    uint64_t* acc_full = empty_bar + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_bias = reinterpret_cast<float*>(misc + 256);  // [BN]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_n = (N + BN - 1) / BN;
    const int n0 = (blockIdx.x % tiles_n) * BN;
    const int m0 = (blockIdx.x / tiles_n) * 2 * BM;
    const int num_kb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_full, 1);
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
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            // weights do not depend on the previous kernel: fetch them before waiting for it
            const int pre = num_kb < STAGES ? num_kb : STAGES;
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&full_bar[i], Cfg::STAGE_BYTES);
                tma_load_2d(smem + i * Cfg::STAGE_BYTES + Cfg::A_BYTES, &tmB, &full_bar[i], i * BK, n0);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(smem + i * Cfg::STAGE_BYTES, &tmA, &full_bar[i], i * BK, m0);
            int s = pre % STAGES, issued = pre;
            uint32_t ph = (pre / STAGES) & 1;
            for (int i = pre; i < num_kb; ++i) {
                if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_PRODUCER);
                    break;
                }
                mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
                tma_load_2d(smem + s * Cfg::STAGE_BYTES, &tmA, &full_bar[s], i * BK, m0);
                tma_load_2d(smem + s * Cfg::STAGE_BYTES + Cfg::A_BYTES, &tmB, &full_bar[s], i * BK, n0);
                ++issued;
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (*abort_flag) {
                // let copies in flight land before shared memory is reused or released
                for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
                    for (uint32_t sp = 0; sp < ET_SPIN_LIMIT; ++sp)
                        if (mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(BM, BN, 0, 0);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int i = 0; i < num_kb; ++i) {
                if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                    report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_MMA);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024, SWZ_128B);
                    const uint32_t acc = (i | k) != 0 ? 1u : 0u;
                    mma_f16_ss(tmem_base, make_smem_desc(a_addr + k * 32, 16, 1024, SWZ_128B), bd,
                               idesc, acc);
                    mma_f16_ss(tmem_base + BN,
                               make_smem_desc(a_addr + A_STAGE_BYTES + k * 32, 16, 1024, SWZ_128B), bd,
                               idesc, acc);
                }
                mma_commit(&empty_bar[s]);
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (ok) mma_commit(acc_full);
        }
    } else {
        // ---------------- epilogue: both accumulators -> staging -> global ----------------
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int et = threadIdx.x - 64;
        constexpr int NCHUNK = BN / 32;
        for (int i = et; i < BN; i += EPI_THREADS) {
            const int n = n0 + i;
            s_bias[i] = (g.bias != nullptr && n < N) ? __half2float(__ldg(g.bias + n)) : 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        pdl_wait();  // outputs may still be read by the previous kernel
        bool ok = mbar_wait_bounded(acc_full, 0, abort_flag);
        if (!ok) report_error(err_word, abort_flag, DEV_TIMEOUT_GEMM_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
#pragma unroll 1
            for (int sub = 0; sub < 2; ++sub) {
                const int row0 = m0 + sub * BM + q * 32;
                if (row0 >= M) continue;  // this quadrant's rows lie past the problem (warp-uniform)
                const uint32_t lane_addr =
                    tmem_base + sub * BN + (static_cast<uint32_t>(q * 32) << 16);
                uint8_t* stage_base = smem + sub * (BN * 256);
                // 64-column groups alternate between the quadrant's two warps, the other way
                // round for the second accumulator so that both warps get the same share
                int my_chunks[NCHUNK];
                int n_my = 0;
#pragma unroll
                for (int ch = 0; ch < NCHUNK; ++ch)
                    if ((((ch >> 1) + sub) & 1) == half && n0 + ch * 32 < N) my_chunks[n_my++] = ch;

                auto finish_chunk = [&](int ch, const uint32_t (&r)[32]) {
                    uint8_t* tile = stage_base + (q * (BN / 64) + (ch >> 1)) * 4096;
                    uint8_t* srow = tile + lane * 128;
                    const float* b32 = s_bias + ch * 32;
                    stage_f16_chunk<ACT>(r, b32, srow, ch & 1, lane);
                    if ((ch & 1) || n0 + ch * 32 + 32 >= N) {  // the 64-column group is complete
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) tma_store_2d(&tmY, tile, n0 + (ch >> 1) * 64, row0);
                    }
                };

                uint32_t ra[32], rb[32];
                if (n_my > 0) {
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
            }
            if (lane == 0) {
                tma_store_commit();
                tma_store_wait_read();
            }
        }
    }

    pdl_wait();  // no CTA may retire before the kernels it depends on have completed
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int BN, int STAGES, int ACT>
int launch_tall_act(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
                    const GemmArgs& args, cudaStream_t stream) {
    using Cfg = TallCfg<BN, STAGES>;
    auto kern = gemm_tall_kernel<BN, STAGES, ACT>;
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::SMEM_BYTES) != cudaSuccess)
            return ET_ERR_CUDA;
        attr_set[dev] = true;
    }
    const long tiles = static_cast<long>((args.N + BN - 1) / BN) * ((args.M + 2 * BM - 1) / (2 * BM));
    return launch_kernel(kern, dim3(static_cast<unsigned>(tiles)), dim3(GEMM_THREADS),
                         Cfg::SMEM_BYTES, stream, tmA, tmB, tmY, args) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

template <int BN, int STAGES>
int launch_tall_cfg(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
                    const GemmArgs& args, cudaStream_t stream) {
    if (args.act == ET_ACT_GELU)
        return launch_tall_act<BN, STAGES, ET_ACT_GELU>(tmA, tmB, tmY, args, stream);
    if (args.act == ET_ACT_RELU)
        return launch_tall_act<BN, STAGES, ET_ACT_RELU>(tmA, tmB, tmY, args, stream);
    return launch_tall_act<BN, STAGES, ET_ACT_NONE>(tmA, tmB, tmY, args, stream);
}

}  // namespace

// bn: 128, 192 or 256.  Same contract as launch_gemm_f16 without an index list.
int launch_gemm_tall_f16(const __half* X, int ldx, const __half* W, int ldw, const __half* bias,
                         __half* Y, int ldy, int M, int N, int K, int act, int bn,
                         cudaStream_t stream) {
    if (!X || !W || !Y || M <= 0 || N <= 0 || K <= 0) return ET_ERR_INVALID_ARG;
    if (act < ET_ACT_NONE || act > ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    if (!aligned16(X) || !aligned16(W) || !aligned16(Y) || (bias && !aligned16(bias)))
        return ET_ERR_ALIGNMENT;
    if (ldx % 8 || ldw % 8 || K % 8 || N % 8 || ldy % 8) return ET_ERR_SHAPE;
    if (bn != 128 && bn != 192 && bn != 256) return ET_ERR_INVALID_ARG;
    if (!device_error_word()) return ET_ERR_NO_DEVICE;
    CUtensorMap tmA, tmB, tmY;
    int st;
    if ((st = gemm::encode_operand(&tmA, X, ldx, M, K, 2 * gemm::BM)) != ET_OK) return st;
    if ((st = gemm::encode_operand(&tmB, W, ldw, N, K, bn)) != ET_OK) return st;
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
    if (bn == 256) return launch_tall_cfg<256, 3>(tmA, tmB, tmY, a, stream);
    if (bn == 192) return launch_tall_cfg<192, 3>(tmA, tmB, tmY, a, stream);
    return launch_tall_cfg<128, 4>(tmA, tmB, tmY, a, stream);
}

}  // namespace et
