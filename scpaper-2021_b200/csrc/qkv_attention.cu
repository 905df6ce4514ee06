// Fused Q/K/V projection + self-attention for short sequences: one CTA per (sequence, head)
// computes that head's Q, K and V (128 tokens x 192 features, K = hidden) with tcgen05.mma
// into tensor memory, converts them (bias added) to fp16 operand tiles in shared memory - the
// same 128-byte-swizzled layout a TMA load of a stored Q / K / V block would produce - and runs
// S = Q.K^T, the softmax and O = P.V on them without the projected activations ever leaving
// the SM.  It replaces the fused-QKV Linear followed by the attention launch
// (reference Attention/Attention.h:204-266) for seq <= 128 and 64-wide heads; the separate
// kernels serve every other shape.
//
// Roles: warp 0 = TMA producer (X block and the head's three 64-row weight slices per K block),
// warp 1 = MMA issuer, warps 2-9 = conversion of the projection, then softmax and output (two
// warps per tensor-memory lane quadrant, 64 keys of a query row each).  Shared memory: a
// two-stage ring (2 x 40 KB) that is reused, once the projection's products are complete, for
// the Q, K, V tiles (3 x 16 KB) and the probability tile (32 KB, later the output staging
// tile); 256 tensor-memory columns: Q | K | V accumulators in [0, 192), then S in [0, 128) and
// O in [192, 256).  Two CTAs fit one SM.  All waits are bounded.
#include <math.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "kernels.h"

namespace et {

// Bring-up aid: with -DET_TIMELINE every CTA records clock64() at a few points of its life.
#ifdef ET_TIMELINE
__device__ long long et_qa_timeline[4096 * 16];
#define QA_TL(slot)                                                                      \
    do {                                                                                 \
        et_qa_timeline[(blockIdx.y * gridDim.x + blockIdx.x) * 16 + (slot)] = clock64(); \
    } while (0)
#else
#define QA_TL(slot) ((void)0)
#endif

namespace {

constexpr int QA_THREADS = 320;
constexpr int QA_SM_THREADS = 256;
constexpr int QA_ATOM = 128 * 128;               // 128 rows x 64 fp16
constexpr int QA_STAGE = QA_ATOM + 3 * 64 * 128; // X block + three weight slices = 40 KB
constexpr int QA_STAGES = 2;
constexpr int QA_RING = QA_STAGES * QA_STAGE;    // 80 KB = Q + K + V + 2 atoms of P
constexpr int QA_MISC = 256 + 192 * 4 + 6 * 128 * 4;
constexpr int QA_SMEM = QA_RING + QA_MISC + 1024;
constexpr int QA_TMEM = 256;
static_assert(QA_RING == 5 * QA_ATOM, "ring must hold Q, K, V and two atoms of P");
static_assert(QA_SMEM <= 113 * 1024, "two CTAs per SM");

struct QkvAttnArgs {
    const __half* bias;  // [2 * kdim + vdim] or null
    const __half* mask;
    const int* valid_len;
    int seq, hidden, kdim;
    int mask_kind;
    float scale_log2;
    int* err_word;
};

// MASK: the mask kind, compiled in (run-time branches around the softmax code cost issue
// efficiency, as they did in the GEMM epilogues).
template <int MASK>
__global__ void __launch_bounds__(QA_THREADS, 2)
qkv_attention_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ CUtensorMap tmZ, const QkvAttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = smem;                  // the tiles alias the ring once the projection is done
    uint8_t* sK = smem + QA_ATOM;
    uint8_t* sV = smem + 2 * QA_ATOM;
    uint8_t* sP = smem + 3 * QA_ATOM;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + QA_RING);
    uint64_t* full_bar = bars;       // [2]
    uint64_t* empty_bar = bars + 2;  // [2]
    uint64_t* proj_full = bars + 4;
    uint64_t* qkv_ready = bars + 5;
    uint64_t* s_full = bars + 6;
    uint64_t* p_full = bars + 7;
    uint64_t* o_full = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_bias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [192]
    float* s_x = s_bias + 192;  // max exchange [2][128], sum exchange [2][128]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int h = blockIdx.x;
    const int b = blockIdx.y;
    const int nkb = (a.hidden + 63) >> 6;

    int kv_len = a.seq;
    if (MASK == ET_MASK_PADDING) {
        kv_len = a.valid_len[b];
        kv_len = kv_len < 0 ? 0 : (kv_len > a.seq ? a.seq : kv_len);
    }

    if (threadIdx.x == 0) {
        QA_TL(0);
#ifdef ET_TIMELINE
        {
            unsigned smid;
            unsigned long long gt;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
            et_qa_timeline[(blockIdx.y * gridDim.x + blockIdx.x) * 16 + 13] = smid;
            et_qa_timeline[(blockIdx.y * gridDim.x + blockIdx.x) * 16 + 14] = (long long)gt;
        }
#endif
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmW);
        for (int s = 0; s < QA_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(proj_full, 1);
        mbar_init(qkv_ready, QA_SM_THREADS);
        mbar_init(s_full, 1);
        mbar_init(p_full, QA_SM_THREADS);
        mbar_init(o_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, QA_TMEM);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base;
    const uint32_t tmem_O = tmem_base + 192;
    pdl_launch_dependents();
    if (threadIdx.x == 0) QA_TL(1);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            auto load_w = [&](int kb, int s) {
                uint8_t* sB = smem + s * QA_STAGE + QA_ATOM;
                tma_load_2d(sB, &tmW, &full_bar[s], kb * 64, h * 64);
                tma_load_2d(sB + 8192, &tmW, &full_bar[s], kb * 64, a.kdim + h * 64);
                tma_load_2d(sB + 16384, &tmW, &full_bar[s], kb * 64, 2 * a.kdim + h * 64);
            };
            // weights do not depend on the previous kernel: fetch them before waiting for it
            const int pre = nkb < QA_STAGES ? nkb : QA_STAGES;
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&full_bar[i], QA_STAGE);
                load_w(i, i);
            }
            pdl_wait();
            QA_TL(2);
            for (int i = 0; i < pre; ++i)
                tma_load_3d(smem + i * QA_STAGE, &tmX, &full_bar[i], i * 64, 0, b);
            int s = pre % QA_STAGES;
            uint32_t ph = (pre / QA_STAGES) & 1;
            int issued = pre;
            for (int i = pre; i < nkb; ++i) {
                if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) {
                    report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_PRODUCER);
                    break;
                }
                mbar_arrive_expect_tx(&full_bar[s], QA_STAGE);
                tma_load_3d(smem + s * QA_STAGE, &tmX, &full_bar[s], i * 64, 0, b);
                load_w(i, s);
                ++issued;
                if (++s == QA_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            QA_TL(3);
            if (*abort_flag) {
                // let copies in flight land before the ring is reused or released
                for (int i = issued > QA_STAGES ? issued - QA_STAGES : 0; i < issued; ++i)
                    for (uint32_t sp = 0; sp < ET_SPIN_LIMIT; ++sp)
                        if (mbar_try_wait(&full_bar[i % QA_STAGES], (i / QA_STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc_p = make_idesc_f16(128, 192, 0, 0);
            constexpr uint32_t idesc_s = make_idesc_f16(128, 128, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_f16(128, 64, 0, 1);  // V is MN-major
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) {
                    report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if (i == 0) QA_TL(4);
                const uint32_t a_addr = smem_u32(smem + s * QA_STAGE);
                const uint32_t b_addr = a_addr + QA_ATOM;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_f16_ss(tmem_base, make_smem_desc(a_addr + k * 32, 16, 1024, SWZ_128B),
                               make_smem_desc(b_addr + k * 32, 16, 1024, SWZ_128B), idesc_p,
                               (i | k) != 0 ? 1u : 0u);
                mma_commit(&empty_bar[s]);
                if (++s == QA_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (ok) {
                mma_commit(proj_full);
                QA_TL(5);
                ok = mbar_wait_bounded(qkv_ready, 0, abort_flag);
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
            }
            if (ok) {
                tc_fence_after_sync();
                const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV),
                               p_addr = smem_u32(sP);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    mma_f16_ss(tmem_S, make_smem_desc(q_addr + kk * 32, 16, 1024, SWZ_128B),
                               make_smem_desc(k_addr + kk * 32, 16, 1024, SWZ_128B), idesc_s,
                               kk != 0 ? 1u : 0u);
                mma_commit(s_full);
                ok = mbar_wait_bounded(p_full, 0, abort_flag);
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
                if (ok) {
                    tc_fence_after_sync();
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t p_off = (kk >> 2) * QA_ATOM + (kk & 3) * 32;
                        // V tile: 16 keys = two groups of 8 rows of 128 bytes (SBO = 1024)
                        mma_f16_ss(tmem_O, make_smem_desc(p_addr + p_off, 16, 1024, SWZ_128B),
                                   make_smem_desc(v_addr + kk * 2048, QA_ATOM, 1024, SWZ_128B),
                                   idesc_o, kk != 0 ? 1u : 0u);
                    }
                    mma_commit(o_full);
                }
            }
        }
    } else {
        // ---------------- conversion, softmax, output ----------------
        const int qd = warp & 3;         // tensor-memory lane quadrant
        const int hf = (warp - 2) >> 2;  // which half of the columns / keys this warp owns
        const int r = qd * 32 + lane;    // token row of the CTA tile = position in the sequence
        const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
        const float NINF = -INFINITY;
        const int et_i = threadIdx.x - 64;
        // bias of this head's Q | K | V features
        if (et_i < 192) {
            const int grp = et_i >> 6, f = et_i & 63;
            const int idx = (grp == 0 ? 0 : (grp == 1 ? a.kdim : 2 * a.kdim)) + h * 64 + f;
            s_bias[et_i] = a.bias != nullptr ? __half2float(__ldg(a.bias + idx)) : 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(QA_SM_THREADS) : "memory");
        pdl_wait();  // Z may still be read by an earlier kernel

        bool ok = mbar_wait_bounded(proj_full, 0, abort_flag);
        if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
            if (threadIdx.x == 64) QA_TL(6);
            // this warp's three 32-column chunks of Q | K | V: accumulator -> fp16 operand tile
            uint32_t ra[32], rb[32];
            const int c0 = hf * 3;
            tmem_ld32(tmem_base + lane_off + c0 * 32, ra);
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int ch = c0 + i;
                uint8_t* srow = smem + (ch >> 1) * QA_ATOM + r * 128;
                if (i & 1) {
                    tmem_ld_wait_regs(rb);
                    if (i + 1 < 3) tmem_ld32(tmem_base + lane_off + (ch + 1) * 32, ra);
                    gemm::stage_f16_chunk<ET_ACT_NONE>(rb, s_bias + ch * 32, srow, ch & 1, lane);
                } else {
                    tmem_ld_wait_regs(ra);
                    if (i + 1 < 3) tmem_ld32(tmem_base + lane_off + (ch + 1) * 32, rb);
                    gemm::stage_f16_chunk<ET_ACT_NONE>(ra, s_bias + ch * 32, srow, ch & 1, lane);
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();  // the tiles are read by the tensor core
            mbar_arrive(qkv_ready);
            if (threadIdx.x == 64) QA_TL(7);

            ok = mbar_wait_bounded(s_full, 0, abort_flag);
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_SOFTMAX);
        }
        ok = __all_sync(0xffffffffu, ok);

        float* xmax = s_x;            // [2 halves][128 rows]
        float* xsum = s_x + 2 * 128;  // [2 halves][128 rows]
        uint32_t v0[32], v1[32];
        float mx = NINF;
        bool need_mask = false;
        if (ok) {
            tc_fence_after_sync();
            if (threadIdx.x == 64) QA_TL(8);
            tmem_ld32(tmem_S + lane_off + hf * 64, v0);
            tmem_ld32(tmem_S + lane_off + hf * 64 + 32, v1);
            tmem_ld_wait_regs(v0);
            tmem_ld_wait_regs(v1);
            const int kbase = hf * 64;
            need_mask = (128 > kv_len) || (MASK == ET_MASK_ADDITIVE) ||
                        (MASK == ET_MASK_CAUSAL);
            if (need_mask) {
                const __half* mrow = (MASK == ET_MASK_ADDITIVE && r < a.seq)
                                         ? a.mask + static_cast<size_t>(r) * a.seq
                                         : nullptr;
                auto fix = [&](uint32_t raw, int kc) -> uint32_t {
                    float s = __uint_as_float(raw) * a.scale_log2;
                    if (kc >= kv_len || (MASK == ET_MASK_CAUSAL && kc > r)) s = NINF;
                    else if (mrow) s += __half2float(__ldg(mrow + kc)) * 1.4426950408889634f;
                    mx = fmaxf(mx, s);
                    return __float_as_uint(s);
                };
#pragma unroll
                for (int i = 0; i < 32; ++i) v0[i] = fix(v0[i], kbase + i);
#pragma unroll
                for (int i = 0; i < 32; ++i) v1[i] = fix(v1[i], kbase + 32 + i);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    mx = fmaxf(mx, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
                mx *= a.scale_log2;
            }
            xmax[hf * 128 + r] = mx;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(QA_SM_THREADS) : "memory");
        float l_part = 0.f;
        if (ok) {
            mx = fmaxf(mx, xmax[(hf ^ 1) * 128 + r]);
            const float neg_m = (mx == NINF) ? 0.f : -mx;
            uint8_t* prow = sP + hf * QA_ATOM + r * 128;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t raw = g < 4 ? v0[g * 8 + i] : v1[(g - 4) * 8 + i];
                    const float arg = need_mask ? __uint_as_float(raw) + neg_m
                                                : fmaf(__uint_as_float(raw), a.scale_log2, neg_m);
                    p[i] = exp2_approx(arg);
                    l_part += p[i];
                }
                uint4 pk;
                pk.x = pack_half2(p[0], p[1]);
                pk.y = pack_half2(p[2], p[3]);
                pk.z = pack_half2(p[4], p[5]);
                pk.w = pack_half2(p[6], p[7]);
                *reinterpret_cast<uint4*>(prow + ((g ^ (r & 7)) * 16)) = pk;
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            mbar_arrive(p_full);
            if (threadIdx.x == 64) QA_TL(9);
            xsum[hf * 128 + r] = l_part;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(QA_SM_THREADS) : "memory");
        if (ok) {
            const float l_run = l_part + xsum[(hf ^ 1) * 128 + r];
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            ok = mbar_wait_bounded(o_full, 0, abort_flag);
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_SOFTMAX);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after_sync();
                if (threadIdx.x == 64) QA_TL(10);
                // this warp's 32 of the 64 output columns -> staging tile (P is dead by now)
                uint32_t o[32];
                tmem_ld32(tmem_O + lane_off + hf * 32, o);
                tmem_ld_wait_regs(o);
                uint8_t* srow = sP + r * 128;
#pragma unroll
                for (int gq = 0; gq < 4; ++gq) {
                    uint4 w;
                    w.x = pack_half2(__uint_as_float(o[gq * 8 + 0]) * inv, __uint_as_float(o[gq * 8 + 1]) * inv);
                    w.y = pack_half2(__uint_as_float(o[gq * 8 + 2]) * inv, __uint_as_float(o[gq * 8 + 3]) * inv);
                    w.z = pack_half2(__uint_as_float(o[gq * 8 + 4]) * inv, __uint_as_float(o[gq * 8 + 5]) * inv);
                    w.w = pack_half2(__uint_as_float(o[gq * 8 + 6]) * inv, __uint_as_float(o[gq * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(srow + (((hf * 4 + gq) ^ (r & 7)) * 16)) = w;
                }
                fence_proxy_async_smem();
            }
        }
        // both warps of the quadrant have filled their halves of the 32 staged rows
        asm volatile("bar.sync %0, 64;" ::"r"(2 + qd) : "memory");
        if (ok && hf == 0 && lane == 0 && qd * 32 < a.seq) {
            tma_store_3d(&tmZ, sP + qd * 32 * 128, h * 64, qd * 32, b);
            tma_store_commit();
            tma_store_wait_read();
            if (qd == 0) QA_TL(11);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) QA_TL(12);
    if (warp == 1) tmem_dealloc(tmem_base, QA_TMEM);
}

}  // namespace

bool qkv_attention_applies(int seq, int nhead, int kdim, int vdim) {
    return seq > 0 && seq <= 128 && nhead > 0 && kdim == nhead * 64 && vdim == nhead * 64;
}

// Z[b, :, h * 64 ..] = softmax(Q_h K_h^T * scale + mask) V_h with [Q | K | V] = X Wqkv^T + b.
int launch_qkv_attention(const __half* X, const __half* Wqkv, const __half* bqkv, __half* Z,
                         int batch, int seq, int hidden, int nhead, int kdim, int vdim, int ldz,
                         int mask_kind, const __half* mask, const int* valid_len, float scale,
                         cudaStream_t stream) {
    if (!X || !Wqkv || !Z || batch <= 0 || seq <= 0 || hidden <= 0 || nhead <= 0)
        return ET_ERR_INVALID_ARG;
    if (mask_kind < ET_MASK_NONE || mask_kind > ET_MASK_ADDITIVE) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_ADDITIVE && !mask) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_PADDING && !valid_len) return ET_ERR_INVALID_ARG;
    if (!(scale > 0.f)) return ET_ERR_INVALID_ARG;
    if (!qkv_attention_applies(seq, nhead, kdim, vdim)) return ET_ERR_SHAPE;
    if (hidden % 8 || ldz % 8 || ldz < vdim || batch > 65535) return ET_ERR_SHAPE;
    if (!aligned16(X) || !aligned16(Wqkv) || !aligned16(Z) || (bqkv && !aligned16(bqkv)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;

    CUtensorMap tmX, tmW, tmZ;
    int st;
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(hidden), static_cast<uint64_t>(seq),
                                  static_cast<uint64_t>(batch)};
        const uint64_t strides[2] = {static_cast<uint64_t>(hidden) * 2,
                                     static_cast<uint64_t>(hidden) * 2 * static_cast<uint64_t>(seq)};
        const uint32_t box[3] = {64, 128, 1};
        if ((st = make_tensor_map_f16(&tmX, X, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != ET_OK)
            return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(hidden), static_cast<uint64_t>(2 * kdim + vdim)};
        const uint64_t strides[1] = {static_cast<uint64_t>(hidden) * 2};
        const uint32_t box[2] = {64, 64};
        if ((st = make_tensor_map_f16(&tmW, Wqkv, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != ET_OK)
            return st;
    }
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(vdim), static_cast<uint64_t>(seq),
                                  static_cast<uint64_t>(batch)};
        const uint64_t strides[2] = {static_cast<uint64_t>(ldz) * 2,
                                     static_cast<uint64_t>(ldz) * 2 * static_cast<uint64_t>(seq)};
        const uint32_t box[3] = {64, 32, 1};
        if ((st = make_tensor_map_f16(&tmZ, Z, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != ET_OK)
            return st;
    }
    int dev = 0;
    cudaGetDevice(&dev);
    auto go = [&](auto kern, int slot, const QkvAttnArgs& args) -> int {
        static std::atomic<bool> attr_set[4][64] = {};
        if (dev >= 0 && dev < 64 && !attr_set[slot][dev]) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, QA_SMEM) !=
                cudaSuccess)
                return ET_ERR_CUDA;
            attr_set[slot][dev] = true;
        }
        return launch_kernel(kern, dim3(nhead, batch), dim3(QA_THREADS), QA_SMEM, stream, tmX, tmW,
                             tmZ, args) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    };
    QkvAttnArgs a;
    a.bias = bqkv;
    a.mask = mask;
    a.valid_len = valid_len;
    a.seq = seq;
    a.hidden = hidden;
    a.kdim = kdim;
    a.mask_kind = mask_kind;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.err_word = err;
    switch (mask_kind) {
        case ET_MASK_CAUSAL: return go(qkv_attention_kernel<ET_MASK_CAUSAL>, 1, a);
        case ET_MASK_PADDING: return go(qkv_attention_kernel<ET_MASK_PADDING>, 2, a);
        case ET_MASK_ADDITIVE: return go(qkv_attention_kernel<ET_MASK_ADDITIVE>, 3, a);
        default: return go(qkv_attention_kernel<ET_MASK_NONE>, 0, a);
    }
}

}  // namespace et

extern "C" {

int et_qkv_attention_fwd(const et_half* X, const et_half* Wqkv, const et_half* bqkv, et_half* Z,
                         int batch, int seq, int hidden, int nhead, int kdim, int vdim,
                         int mask_kind, const et_half* mask, const int32_t* valid_len, float scale,
                         et_stream stream) {
    return et::launch_qkv_attention(
        reinterpret_cast<const __half*>(X), reinterpret_cast<const __half*>(Wqkv),
        reinterpret_cast<const __half*>(bqkv), reinterpret_cast<__half*>(Z), batch, seq, hidden,
        nhead, kdim, vdim, vdim, mask_kind, reinterpret_cast<const __half*>(mask), valid_len, scale,
        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
