// Body of the on-the-fly attention kernel for one (sequence, head, 128-query block), shared by
// the stand-alone kernel (attention.cu) and the kernel that also runs the output projection
// (attention_fuse_o.cu).
//
// One CTA owns 128 queries of one (sequence, head).  Warp 0 streams Q once and then K / V
// blocks of 128 keys with TMA (3-D tensor maps {feature, position, sequence}, so positions
// past the end of a sequence are zero-filled and never read the next sequence).  One
// thread of warp 1 issues S = Q.K^T (M=128, N=128) into tensor memory.  Eight softmax warps
// share the 128 x 128 score block: two per tensor-memory lane quadrant, each thread owning
// 64 keys of one query row, which it reads from tensor memory ONCE and keeps in registers.
// The two halves of a row exchange their maxima through shared memory, then each thread
// computes exp2 (with log2(e)/sqrt(dh) folded into one FMA), keeps a running max / partial
// sum (online softmax across key blocks), writes its fp16 probabilities into the
// 128-byte-swizzled shared-memory tile that is the A operand of the second product and
// rescales its share of the output accumulator when the running max was raised (only when a
// block exceeds it by more than 2^8, so a few times per row).  The MMA thread issues the next
// block's Q.K^T ahead of O += P.V (V consumed directly in its row-major, MN-major layout), so
// the scores of block j+1 are ready when the softmax warps finish block j.  After
// the last block the row sums are combined, each thread scales its share of the output
// columns and the tile leaves through a swizzled staging buffer and TMA stores.
// All waits are bounded.
#pragma once
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace et {
namespace attn {

// Optional per-CTA timestamps for bring-up builds (-DET_TIMELINE); compiled out otherwise.
#undef ET_TL
#ifdef ET_TIMELINE
static __device__ long long et_attn_timeline[65536];
#define ET_TL(slot)                                                                       \
    et_attn_timeline[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + \
                     (slot)] = clock64()
#else
#define ET_TL(slot) ((void)0)
#endif

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int SM_WARPS = 8;                      // softmax / output warps
constexpr int SM_THREADS = 32 * SM_WARPS;
constexpr int ATT_THREADS = 64 + SM_THREADS;
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows x 64 fp16, one 128-byte-swizzled atom
constexpr int TMEM_COLS_ATT = 256;     // S: columns [0,128), O: columns [128, 128 + v_n)
constexpr int EXTRA_BYTES = 256 + 6 * 128 * 4;   // barriers + max / sum exchange arrays

// The running maximum is only raised when a block's maximum exceeds it by more than this many
// powers of two: probabilities then stay below 2^8 (exact in fp16's range, fp32 sums), the final
// division by the row sum removes the common factor, and the output accumulator is rescaled
// in tensor memory a few times per row instead of after most key blocks.
constexpr float RESCALE_SLACK = 8.0f;

// 64 scores of one query row -> fp16 probabilities in the swizzled P tile; returns their sum.
// SCALED: the scores were already scaled and masked in place (log2 domain).
template <bool SCALED>
__device__ __forceinline__ float store_probabilities(const uint32_t (&v0)[32],
                                                     const uint32_t (&v1)[32], float scale_log2,
                                                     float neg_m, uint8_t* prow, int r) {
    float rowsum = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float raw = __uint_as_float(g < 4 ? v0[g * 8 + i] : v1[(g - 4) * 8 + i]);
            p[i] = exp2_approx(SCALED ? raw + neg_m : fmaf(raw, scale_log2, neg_m));
            rowsum += p[i];
        }
        uint4 pk;
        pk.x = pack_half2(p[0], p[1]);
        pk.y = pack_half2(p[2], p[3]);
        pk.z = pack_half2(p[4], p[5]);
        pk.w = pack_half2(p[6], p[7]);
        *reinterpret_cast<uint4*>(prow + ((g ^ (r & 7)) * 16)) = pk;
    }
    return rowsum;
}

constexpr int ATT_MAX_UNITS = 16;

struct AttnArgs {
    __half* Z;
    const __half* mask;
    const int* valid_len;
    int ldz;
    int batch, seq, nhead, dh_qk, dh_v;
    int mask_kind;
    float scale_log2;  // scale * log2(e), > 0
    int* err_word;
    // column-compressed V (null for a dense V): feature list and per-head ranges into it
    const int* col_id;
    const int* head_ptr;
    int nva_max;    // 64-feature atoms reserved for a V block in shared memory
    int tmem_cols;  // tensor-memory columns to allocate (256 or 512)
    int tma_out;    // 1: the output tile is written with TMA stores (dense V, dh_v % 64 == 0)
    // Work-unit form (n_units > 0): blockIdx.y selects a unit = (head, first 128-query block);
    // the grid's x extent is the number of query blocks per unit.  Otherwise blockIdx.y is the
    // head and the grid covers every query block.
    int n_units;
    unsigned char unit_head[ATT_MAX_UNITS];
    unsigned short unit_first[ATT_MAX_UNITS];
};

// The work of one CTA: queries [q0, q0 + 128) of head h of sequence b.  `smem` is the CTA's
// 1024-byte-aligned dynamic shared memory.
// MASK: the mask kind, compiled in (keeps the mask bookkeeping out of the registers of the
// kinds that do not need it).
// FUSED == false: the body of a kernel of its own - it allocates and frees tensor memory, owns
// the abort flag and takes part in programmatic dependent launch.
// FUSED == true: one of several pieces of work a CTA runs in turn - tensor memory (tmem_in) and
// the abort flag (abort_in) belong to the caller, the output is complete in global memory (not
// merely read out of the staging tile) when the function returns, and the barriers are
// invalidated at the end so that the next piece of work may lay out shared memory afresh.
template <int MASK, bool FUSED>
__device__ __forceinline__ void attention_cta(const CUtensorMap& tmQ, const CUtensorMap& tmK,
                                              const CUtensorMap& tmV, const CUtensorMap& tmZ,
                                              const AttnArgs& a, uint8_t* smem, int q0, int h, int b,
                                              uint32_t tmem_in, volatile int* abort_in) {
    const int nqa = (a.dh_qk + 63) >> 6;  // 64-feature atoms of Q / K
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + nqa * ATOM_BYTES;
    uint8_t* sV = sK + nqa * ATOM_BYTES;
    uint8_t* sP = sV + a.nva_max * ATOM_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * ATOM_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 2;
    uint64_t* v_full = bars + 3;
    uint64_t* v_empty = bars + 4;
    uint64_t* s_full = bars + 5;
    uint64_t* s_free = bars + 6;
    uint64_t* p_full = bars + 7;
    uint64_t* o_full = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = FUSED ? abort_in : reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_xmax = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // V window of this head: feature offset v_x0 (a multiple of 8 so the TMA start is 16-byte
    // aligned), v_n accumulator columns, of which [v_shift, v_shift + v_cnt) are this head's.
    int v_x0 = h * a.dh_v, v_shift = 0, v_cnt = a.dh_v, v_n = a.dh_v;
    if (a.head_ptr != nullptr) {
        const int c0 = a.head_ptr[h];
        v_cnt = a.head_ptr[h + 1] - c0;
        v_x0 = c0 & ~7;
        v_shift = c0 - v_x0;
        v_n = (v_shift + v_cnt + 15) & ~15;
        v_n = v_n < 16 ? 16 : v_n;
    }
    const int nva = (v_n + 63) >> 6;  // 64-feature atoms of V actually loaded

    int kv_len = a.seq;
    if (MASK == ET_MASK_PADDING) {
        kv_len = a.valid_len[b];
        kv_len = kv_len < 0 ? 0 : (kv_len > a.seq ? a.seq : kv_len);
    }
    int n_kv = (kv_len + BKV - 1) / BKV;
    if (MASK == ET_MASK_CAUSAL) {
        const int last_q = (q0 + BQ - 1 < a.seq ? q0 + BQ - 1 : a.seq - 1);
        const int lim = last_q / BKV + 1;
        n_kv = n_kv < lim ? n_kv : lim;
    }

    if (threadIdx.x == 0) {
        ET_TL(0);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_init(q_full, 1);
        mbar_init(k_full, 1);
        mbar_init(k_empty, 1);
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(s_free, SM_THREADS);
        mbar_init(p_full, SM_THREADS);
        mbar_init(o_full, 1);
        if (!FUSED) *abort_flag = 0;
        fence_barrier_init();
    }
    if (!FUSED && warp == 1) {
        tmem_alloc(tmem_slot, a.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = FUSED ? tmem_in : *tmem_slot;
    const uint32_t tmem_S = tmem_base;
    const uint32_t tmem_O = tmem_base + 128;
    if (threadIdx.x == 0) ET_TL(1);
    if (!FUSED) {
        pdl_launch_dependents();
        pdl_wait();  // Q, K, V come from the previous kernel; Z may still be read by an earlier one
    }

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (n_kv > 0 && elect_one()) {
            mbar_arrive_expect_tx(q_full, nqa * ATOM_BYTES);
            for (int t = 0; t < nqa; ++t)
                tma_load_3d(sQ + t * ATOM_BYTES, &tmQ, q_full, h * a.dh_qk + t * 64, q0, b);
            int k_issued = 0, v_issued = 0;
            for (int j = 0; j < n_kv; ++j) {
                const uint32_t ph = j & 1;
                if (!mbar_wait_bounded_relaxed(k_empty, ph ^ 1, abort_flag)) {
                    report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_PRODUCER);
                    break;
                }
                mbar_arrive_expect_tx(k_full, nqa * ATOM_BYTES);
                for (int t = 0; t < nqa; ++t)
                    tma_load_3d(sK + t * ATOM_BYTES, &tmK, k_full, h * a.dh_qk + t * 64, j * BKV, b);
                ++k_issued;
                if (!mbar_wait_bounded_relaxed(v_empty, ph ^ 1, abort_flag)) {
                    report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_PRODUCER);
                    break;
                }
                mbar_arrive_expect_tx(v_full, nva * ATOM_BYTES);
                for (int t = 0; t < nva; ++t)
                    tma_load_3d(sV + t * ATOM_BYTES, &tmV, v_full, v_x0 + t * 64, j * BKV, b);
                ++v_issued;
                if (j == 0) ET_TL(2);
            }
            if (*abort_flag) {
                // let copies in flight land before shared memory is released
                for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                    if (mbar_try_wait(q_full, 0)) break;
                if (k_issued > 0)
                    for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                        if (mbar_try_wait(k_full, (k_issued - 1) & 1)) break;
                if (v_issued > 0)
                    for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                        if (mbar_try_wait(v_full, (v_issued - 1) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (n_kv > 0 && elect_one()) {
            const uint32_t idesc_s = make_idesc_f16(BQ, BKV, 0, 0);
            const uint32_t idesc_o = make_idesc_f16(BQ, v_n, 0, 1);  // V is MN-major
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV),
                           p_addr = smem_u32(sP);
            bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
            // S_j = Q.K_j^T; the score block is free as soon as the softmax warps hold it in
            // registers, so S_{j+1} is issued BEFORE P_j.V_j and runs under softmax(j).
            auto issue_s = [&](int j) -> bool {
                const uint32_t ph = j & 1;
                if (!(mbar_wait_bounded(k_full, ph, abort_flag) &&
                      mbar_wait_bounded(s_free, ph ^ 1, abort_flag)))
                    return false;
                tc_fence_after_sync();
                const int ksteps = a.dh_qk >> 4;
                for (int kk = 0; kk < ksteps; ++kk) {
                    const uint32_t off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
                    mma_f16_ss(tmem_S, make_smem_desc(q_addr + off, 16, 1024, SWZ_128B),
                               make_smem_desc(k_addr + off, 16, 1024, SWZ_128B), idesc_s,
                               kk != 0 ? 1u : 0u);
                }
                mma_commit(s_full);
                mma_commit(k_empty);
                return true;
            };
            if (ok) {
                ok = issue_s(0);
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
                ET_TL(3);
            }
            for (int j = 0; ok && j < n_kv; ++j) {
                const uint32_t ph = j & 1;
                if (j + 1 < n_kv) ok = issue_s(j + 1);
                ok = ok && mbar_wait_bounded(p_full, ph, abort_flag) &&
                     mbar_wait_bounded(v_full, ph, abort_flag);
                if (!ok) {
                    report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
                    break;
                }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                    const uint32_t p_off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
                    // V tile: 16 keys = two groups of 8 rows of 128 bytes (SBO = 1024); a second
                    // 64-feature atom sits ATOM_BYTES further (LBO).
                    mma_f16_ss(tmem_O, make_smem_desc(p_addr + p_off, 16, 1024, SWZ_128B),
                               make_smem_desc(v_addr + kk * 2048, ATOM_BYTES, 1024, SWZ_128B),
                               idesc_o, (j | kk) != 0 ? 1u : 0u);
                }
                mma_commit(o_full);
                mma_commit(v_empty);
                if (j == 0) ET_TL(7);
            }
            if (FUSED && ok) {
                // the barriers are invalidated after this piece of work: every arrival a commit
                // has scheduled must have happened by then
                ok = mbar_wait_bounded(k_empty, (n_kv - 1) & 1, abort_flag) &&
                     mbar_wait_bounded(v_empty, (n_kv - 1) & 1, abort_flag);
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_MMA);
            }
        }
    } else {
        // ---------------- softmax / output warps ----------------
        const int qd = warp & 3;          // tensor-memory lane quadrant
        const int hf = (warp - 2) >> 2;   // which 64 keys of a block / which share of the output
        const int r = qd * 32 + lane;     // row inside the CTA tile
        const int qrow = q0 + r;          // position inside the sequence
        const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
        const float NINF = -INFINITY;
        // exchange buffers: maxima double-buffered by block parity, sums single
        float* xmax = s_xmax;                 // [2 parities][2 halves][128 rows]
        float* xsum = s_xmax + 2 * 2 * 128;   // [2 halves][128 rows]
        const int nc16 = v_n >> 4;            // 16-column chunks of the output accumulator
        const int csplit = (nc16 + 1) >> 1;
        const int c_begin = hf * csplit;
        const int c_end = (c_begin + csplit) < nc16 ? (c_begin + csplit) : nc16;
        float m_run = NINF, l_part = 0.f;
        bool ok = true;

        // Error handling: a warp whose bounded wait ran out keeps walking the loop (skipping the
        // work) so that every warp executes the same sequence of named barriers.
        for (int j = 0; j < n_kv; ++j) {
            const uint32_t ph = j & 1;
            if (ok) {
                ok = mbar_wait_bounded(s_full, ph, abort_flag);
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_SOFTMAX);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok) {
                asm volatile("bar.sync 1, %0;" ::"n"(SM_THREADS) : "memory");
                continue;
            }
            tc_fence_after_sync();
            if (threadIdx.x == 64 && j == 0) ET_TL(4);

            const int kbase = j * BKV + hf * 64;
            const bool need_mask = (j * BKV + BKV > kv_len) || (MASK == ET_MASK_ADDITIVE) ||
                                   (MASK == ET_MASK_CAUSAL && j * BKV + BKV - 1 > q0);
            // general path: a score scaled and masked (log2 domain)
            const __half* mrow = (MASK == ET_MASK_ADDITIVE && qrow < a.seq)
                                     ? a.mask + static_cast<size_t>(qrow) * a.seq
                                     : nullptr;
            auto score = [&](uint32_t raw, int kc) -> float {
                float s = __uint_as_float(raw) * a.scale_log2;
                if (kc >= kv_len || (MASK == ET_MASK_CAUSAL && kc > qrow)) s = NINF;
                else if (MASK == ET_MASK_ADDITIVE && mrow)
                    s += __half2float(__ldg(mrow + kc)) * 1.4426950408889634f;
                return s;
            };

            // pass 1: the maximum of this thread's 64 scores.  The scores are not kept: they are
            // read from tensor memory again for pass 2 (cheap), which keeps 64 registers free
            // across the exchange and the accumulator rescale.
            float mx = NINF;
            {
                uint32_t v0[32], v1[32];
                tmem_ld32(tmem_S + lane_off + hf * 64, v0);
                tmem_ld32(tmem_S + lane_off + hf * 64 + 32, v1);
                tmem_ld_wait_regs(v0);
                tmem_ld_wait_regs(v1);
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        mx = fmaxf(mx, fmaxf(score(v0[i], kbase + i), score(v1[i], kbase + 32 + i)));
                } else {
                    // fast path: max of the raw scores, the (positive) scale applied once
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        mx = fmaxf(mx, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
                    mx *= a.scale_log2;
                }
            }
            // combine with the other half of the row
            xmax[(ph * 2 + hf) * 128 + r] = mx;
            asm volatile("bar.sync 1, %0;" ::"n"(SM_THREADS) : "memory");
            mx = fmaxf(mx, xmax[(ph * 2 + (hf ^ 1)) * 128 + r]);
            if (threadIdx.x == 64 && j == 0) ET_TL(5);

            // raise the running maximum only when it is -inf or the block exceeds it by more
            // than the slack (both halves of a row take the same decision: same inputs)
            const bool raise = (m_run == NINF) || (mx > m_run + RESCALE_SLACK);
            const float m_new = raise ? fmaxf(m_run, mx) : m_run;
            const float m_use = (m_new == NINF) ? 0.f : m_new;
            const float alpha = raise ? exp2_approx(m_run - m_use) : 1.0f;  // 0 when m_run = -inf

            if (j > 0) {
                // P and O of the previous block must have been consumed / produced
                ok = mbar_wait_bounded(o_full, ph ^ 1, abort_flag);
                if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_SOFTMAX);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) continue;
                tc_fence_after_sync();
                if (!__all_sync(0xffffffffu, alpha == 1.0f)) {
                    for (int c = c_begin; c < c_end; ++c) {
                        uint32_t o[16];
                        tmem_ld16(tmem_O + lane_off + c * 16, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st16(tmem_O + lane_off + c * 16, o);
                    }
                    tmem_st_wait();
                }
            }

            // pass 2: probabilities -> shared memory (A operand of P.V, atom `hf`), partial sum
            uint8_t* prow = sP + hf * ATOM_BYTES + r * 128;
            float rowsum;
            {
                uint32_t v0[32], v1[32];
                tmem_ld32(tmem_S + lane_off + hf * 64, v0);
                tmem_ld32(tmem_S + lane_off + hf * 64 + 32, v1);
                tmem_ld_wait_regs(v0);
                tmem_ld_wait_regs(v1);
                tc_fence_before_sync();
                mbar_arrive(s_free);  // S may be overwritten by the next Q.K^T
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v0[i] = __float_as_uint(score(v0[i], kbase + i));
                        v1[i] = __float_as_uint(score(v1[i], kbase + 32 + i));
                    }
                    rowsum = store_probabilities<true>(v0, v1, a.scale_log2, -m_use, prow, r);
                } else {
                    rowsum = store_probabilities<false>(v0, v1, a.scale_log2, -m_use, prow, r);
                }
            }
            l_part = l_part * alpha + rowsum;
            m_run = m_new;

            tc_fence_before_sync();
            fence_proxy_async_smem();  // P visible to the tensor core's reads
            mbar_arrive(p_full);
            if (threadIdx.x == 64 && j == 0) ET_TL(6);
        }

        // total row sum = the two halves' partial sums
        xsum[hf * 128 + r] = l_part;
        asm volatile("bar.sync 1, %0;" ::"n"(SM_THREADS) : "memory");
        const float l_run = l_part + xsum[(hf ^ 1) * 128 + r];

        if (ok && n_kv > 0) {
            ok = mbar_wait_bounded(o_full, (n_kv - 1) & 1, abort_flag);
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_ATTN_SOFTMAX);
            ok = __all_sync(0xffffffffu, ok);
        }
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        const bool staged = a.tma_out && n_kv > 0;
        __half* zrow = a.Z + (static_cast<size_t>(b) * a.seq + (qrow < a.seq ? qrow : 0)) * a.ldz +
                       static_cast<size_t>(h) * a.dh_v;
        if (ok) {
            tc_fence_after_sync();
            if (threadIdx.x == 64) ET_TL(8);
            if (a.head_ptr != nullptr && qrow < a.seq && hf == 0) {
                // pruned features of this head are zero; kept ones are scattered below
                for (int c = 0; c < (a.dh_v >> 3); ++c)
                    *reinterpret_cast<uint4*>(zrow + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        // orders the zero fill (done by one warp of the quadrant's pair) before the scatter
        asm volatile("bar.sync %0, 64;" ::"r"(2 + qd) : "memory");
        if (ok) {
            for (int c = c_begin; c < c_end; ++c) {
                uint32_t o[16];
                if (n_kv > 0) {
                    tmem_ld16(tmem_O + lane_off + c * 16, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = 0u;
                }
                uint4 w0, w1;
                w0.x = pack_half2(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
                w0.y = pack_half2(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
                w0.z = pack_half2(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
                w0.w = pack_half2(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
                w1.x = pack_half2(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
                w1.y = pack_half2(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
                w1.z = pack_half2(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
                w1.w = pack_half2(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
                if (staged) {
                    // P is dead once the last P.V product has completed: reuse it as the swizzled
                    // staging tile of the output (64-column atoms, 128 bytes per row)
                    uint8_t* srow = sP + (c >> 2) * ATOM_BYTES + r * 128;
                    const int ch = (c & 3) * 2;
                    *reinterpret_cast<uint4*>(srow + ((ch ^ (r & 7)) * 16)) = w0;
                    *reinterpret_cast<uint4*>(srow + (((ch + 1) ^ (r & 7)) * 16)) = w1;
                } else if (qrow < a.seq) {
                    if (a.head_ptr == nullptr) {
                        *reinterpret_cast<uint4*>(zrow + c * 16) = w0;
                        *reinterpret_cast<uint4*>(zrow + c * 16 + 8) = w1;
                    } else {
                        const int* ids = a.col_id + a.head_ptr[h];
                        const __half* hv0 = reinterpret_cast<const __half*>(&w0);
                        const __half* hv1 = reinterpret_cast<const __half*>(&w1);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int k = c * 16 + i - v_shift;  // index into this head's list
                            if (k >= 0 && k < v_cnt)
                                a.Z[(static_cast<size_t>(b) * a.seq + qrow) * a.ldz + __ldg(ids + k)] =
                                    i < 8 ? hv0[i] : hv1[i - 8];
                        }
                    }
                }
            }
            if (staged) fence_proxy_async_smem();
        }
        // both warps of the quadrant have filled their share of the 32 staged rows
        asm volatile("bar.sync %0, 64;" ::"r"(2 + qd) : "memory");
        if (ok && staged && hf == 0 && lane == 0 && q0 + qd * 32 < a.seq) {
            for (int t = 0; t < nva; ++t)
                tma_store_3d(&tmZ, sP + t * ATOM_BYTES + qd * 32 * 128, h * a.dh_v + t * 64,
                             q0 + qd * 32, b);
            tma_store_commit();
            if (FUSED) {
                tma_store_wait_all();  // complete in global memory, not only read out
                fence_proxy_async_global();
            }
            else tma_store_wait_read();
        }
    }

    if (threadIdx.x == 64) ET_TL(9);
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) ET_TL(10);
    if (FUSED) {
        if (threadIdx.x == 0 && !*abort_flag)
            for (int i = 0; i < 9; ++i) mbar_inval(bars + i);
        __syncthreads();  // nobody reuses this memory while the barriers are still alive
    } else if (warp == 1) {
        tmem_dealloc(tmem_base, a.tmem_cols);
    }
}

}  // namespace attn
}  // namespace et
