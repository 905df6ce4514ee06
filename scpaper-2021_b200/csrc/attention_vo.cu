// Attention with the value and output projections pre-multiplied (W_VO = W_V W_O per head):
//   out[t, :] = bias_o + sum_h softmax(scale * Q_h K_h^T + mask)[t, :] . VO_h
// where VO[b][h] = X_b W_VO[h] has the full model width.
//
// One CTA owns 128 queries of one sequence and a chunk of up to 256 output features, whose
// fp32 accumulator lives in tensor memory for the whole kernel: heads are reduced inside the
// accumulator in a fixed order (h = 0, 1, ...), so the result is deterministic and the output
// needs no pre-zeroing (the reference reduces heads with half2 atomics).  Because every
// head has its own softmax normaliser, probabilities are normalised BEFORE the second
// product: for sequences longer than one key block a first pass over the head's key blocks
// computes the row max and sum (scores only), a second pass recomputes the scores, writes
// P = exp2(s - m) / l as the fp16 A operand and accumulates O += P . VO_h[block].
// Roles, TMA layouts and bounded waits are those of attention.cu.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int VO_THREADS = 192;
constexpr int ATOM_BYTES = 128 * 128;
// NC output features per CTA: 256, or 128 / 64 behind a test hook.  A CTA recomputes the scores
// and the softmax of every head whatever its width, so narrower chunks do more work in total
// and spread it over more CTAs.  Tensor memory: scores in columns [0, 128), the accumulator
// behind them.
__host__ __device__ constexpr int vo_tmem_cols(int nc) { return nc <= 128 ? 256 : 512; }

struct VoArgs {
    __half* out;
    const __half* bias_o;
    const __half* mask;
    const int* valid_len;
    int batch, seq, nhead, dh_qk, emdim;
    int mask_kind;
    float scale_log2;
    int* err_word;
};

template <int NC>
__global__ void __launch_bounds__(VO_THREADS, (NC <= 128 ? 2 : 1))
attention_vo_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmVO, const VoArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment computed on the shared-window offset, so that the pointer keeps its
    // shared-memory provenance (plain LDS / STS instead of generic accesses)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int nqa = (a.dh_qk + 63) >> 6;
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + nqa * ATOM_BYTES;
    uint8_t* sVO = sK + nqa * ATOM_BYTES;
    uint8_t* sP = sVO + (NC / 64) * ATOM_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * ATOM_BYTES);
    uint64_t* qk_full = bars + 0;
    uint64_t* qk_empty = bars + 1;
    uint64_t* vo_full = bars + 2;
    uint64_t* vo_empty = bars + 3;
    uint64_t* s_full = bars + 4;
    uint64_t* s_free = bars + 5;
    uint64_t* p_full = bars + 6;
    uint64_t* pv_done = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * BQ;
    const int e0 = blockIdx.y * NC;
    const int b = blockIdx.z;
    const int n_c = (a.emdim - e0) < NC ? (a.emdim - e0) : NC;  // multiple of 16
    const int nca = (n_c + 63) >> 6;

    int kv_len = a.seq;
    if (a.mask_kind == ET_MASK_PADDING) {
        kv_len = a.valid_len[b];
        kv_len = kv_len < 0 ? 0 : (kv_len > a.seq ? a.seq : kv_len);
    }
    int n_kv = (kv_len + BKV - 1) / BKV;
    if (a.mask_kind == ET_MASK_CAUSAL) {
        const int last_q = (q0 + BQ - 1 < a.seq ? q0 + BQ - 1 : a.seq - 1);
        const int lim = last_q / BKV + 1;
        n_kv = n_kv < lim ? n_kv : lim;
    }
    const int passes = n_kv > 1 ? 2 : 1;  // statistics pass only when a row spans several blocks

    if (threadIdx.x == 0) {
        mbar_init(qk_full, 1);
        mbar_init(qk_empty, 1);
        mbar_init(vo_full, 1);
        mbar_init(vo_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(s_free, 128);
        mbar_init(p_full, 128);
        mbar_init(pv_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, vo_tmem_cols(NC));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base;
    const uint32_t tmem_O = tmem_base + 128;
    pdl_launch_dependents();
    pdl_wait();  // every input is produced by earlier kernels on the stream

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (n_kv > 0 && elect_one()) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmVO);
            int t_qk = 0, t_vo = 0;
            bool ok = true;
            for (int h = 0; ok && h < a.nhead; ++h)
                for (int pass = 0; ok && pass < passes; ++pass)
                    for (int j = 0; ok && j < n_kv; ++j) {
                        ok = mbar_wait_bounded(qk_empty, (t_qk & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        mbar_arrive_expect_tx(qk_full, 2 * nqa * ATOM_BYTES);
                        for (int t = 0; t < nqa; ++t) {
                            tma_load_3d(sQ + t * ATOM_BYTES, &tmQ, qk_full, h * a.dh_qk + t * 64, q0, b);
                            tma_load_3d(sK + t * ATOM_BYTES, &tmK, qk_full, h * a.dh_qk + t * 64,
                                        j * BKV, b);
                        }
                        ++t_qk;
                        if (pass == passes - 1) {
                            ok = mbar_wait_bounded(vo_empty, (t_vo & 1) ^ 1, abort_flag);
                            if (!ok) break;
                            mbar_arrive_expect_tx(vo_full, nca * ATOM_BYTES);
                            for (int t = 0; t < nca; ++t)
                                tma_load_3d(sVO + t * ATOM_BYTES, &tmVO, vo_full, e0 + t * 64, j * BKV,
                                            b * a.nhead + h);
                            ++t_vo;
                        }
                    }
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_VO_PRODUCER);
            if (*abort_flag) {
                if (t_qk > 0)
                    for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                        if (mbar_try_wait(qk_full, (t_qk - 1) & 1)) break;
                if (t_vo > 0)
                    for (uint32_t it = 0; it < ET_SPIN_LIMIT; ++it)
                        if (mbar_try_wait(vo_full, (t_vo - 1) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (n_kv > 0 && elect_one()) {
            const uint32_t idesc_s = make_idesc_f16(BQ, BKV, 0, 0);
            const uint32_t idesc_o = make_idesc_f16(BQ, n_c, 0, 1);
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), vo_addr = smem_u32(sVO),
                           p_addr = smem_u32(sP);
            int t_s = 0, t_b = 0;
            bool ok = true;
            for (int h = 0; ok && h < a.nhead; ++h)
                for (int pass = 0; ok && pass < passes; ++pass)
                    for (int j = 0; ok && j < n_kv; ++j) {
                        ok = mbar_wait_bounded(qk_full, t_s & 1, abort_flag) &&
                             mbar_wait_bounded(s_free, (t_s & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after_sync();
                        for (int kk = 0; kk < (a.dh_qk >> 4); ++kk) {
                            const uint32_t off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
                            mma_f16_ss(tmem_S, make_smem_desc(q_addr + off, 16, 1024, SWZ_128B),
                                       make_smem_desc(k_addr + off, 16, 1024, SWZ_128B), idesc_s,
                                       kk != 0 ? 1u : 0u);
                        }
                        mma_commit(s_full);
                        mma_commit(qk_empty);
                        ++t_s;
                        if (pass == passes - 1) {
                            ok = mbar_wait_bounded(p_full, t_b & 1, abort_flag) &&
                                 mbar_wait_bounded(vo_full, t_b & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after_sync();
#pragma unroll
                            for (int kk = 0; kk < BKV / 16; ++kk) {
                                const uint32_t p_off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
                                mma_f16_ss(tmem_O,
                                           make_smem_desc(p_addr + p_off, 16, 1024, SWZ_128B),
                                           make_smem_desc(vo_addr + kk * 2048, ATOM_BYTES, 1024,
                                                          SWZ_128B),
                                           idesc_o, (t_b | kk) != 0 ? 1u : 0u);
                            }
                            mma_commit(pv_done);
                            mma_commit(vo_empty);
                            ++t_b;
                        }
                    }
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_VO_MMA);
        }
    } else {
        // ---------------- softmax / output warps ----------------
        const int qd = warp & 3;
        const int r = qd * 32 + lane;
        const int qrow = q0 + r;
        const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
        const float NINF = -INFINITY;
        const __half* mrow = (a.mask_kind == ET_MASK_ADDITIVE && qrow < a.seq)
                                 ? a.mask + static_cast<size_t>(qrow) * a.seq
                                 : nullptr;
        int t_s = 0, t_b = 0;
        bool ok = true;

        auto score = [&](uint32_t raw, int kc) -> float {
            if (kc >= kv_len || (a.mask_kind == ET_MASK_CAUSAL && kc > qrow)) return NINF;
            float s = __uint_as_float(raw) * a.scale_log2;
            if (mrow) s += __half2float(__ldg(mrow + kc)) * 1.4426950408889634f;
            return s;
        };
        // running max / sum of one key block (reads S twice: max, then sum)
        auto block_stats = [&](int kbase, float& m_run, float& l_run) {
            float mx = NINF;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_S + lane_off + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, score(v[i], kbase + c * 32 + i));
            }
            const float m_new = fmaxf(m_run, mx);
            const float m_use = (m_new == NINF) ? 0.f : m_new;
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_S + lane_off + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sum += exp2_approx(score(v[i], kbase + c * 32 + i) - m_use);
            }
            l_run = l_run * exp2_approx(m_run - m_use) + sum;
            m_run = m_new;
        };

        for (int h = 0; ok && h < a.nhead; ++h) {
            float m_run = NINF, l_run = 0.f;
            if (passes == 2) {
                for (int j = 0; j < n_kv; ++j) {
                    ok = mbar_wait_bounded(s_full, t_s & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    block_stats(j * BKV, m_run, l_run);
                    tc_fence_before_sync();
                    mbar_arrive(s_free);
                    ++t_s;
                }
                if (!ok) break;
            }
            for (int j = 0; j < n_kv; ++j) {
                ok = mbar_wait_bounded(s_full, t_s & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                if (passes == 1) block_stats(j * BKV, m_run, l_run);
                const float m_use = (m_run == NINF) ? 0.f : m_run;
                const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
                if (t_b > 0) {
                    ok = mbar_wait_bounded(pv_done, (t_b - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const int kbase = j * BKV;
#pragma unroll 1
                for (int c = 0; c < BKV / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_S + lane_off + c * 32, v);
                    tmem_ld_wait();
                    float p[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        p[i] = exp2_approx(score(v[i], kbase + c * 32 + i) - m_use) * inv;
                    uint8_t* prow = sP + (c >> 1) * ATOM_BYTES + r * 128;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 pk;
                        pk.x = pack_half2(p[g * 8 + 0], p[g * 8 + 1]);
                        pk.y = pack_half2(p[g * 8 + 2], p[g * 8 + 3]);
                        pk.z = pack_half2(p[g * 8 + 4], p[g * 8 + 5]);
                        pk.w = pack_half2(p[g * 8 + 6], p[g * 8 + 7]);
                        const int chunk = ((c & 1) * 4 + g) ^ (r & 7);
                        *reinterpret_cast<uint4*>(prow + chunk * 16) = pk;
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(s_free);
                fence_proxy_async_smem();
                mbar_arrive(p_full);
                ++t_s;
                ++t_b;
            }
        }
        if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_VO_SOFTMAX);

        if (ok && t_b > 0) {
            ok = mbar_wait_bounded(pv_done, (t_b - 1) & 1, abort_flag);
            if (!ok) report_error(a.err_word, abort_flag, DEV_TIMEOUT_VO_SOFTMAX);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after_sync();
            __half* orow = a.out + (static_cast<size_t>(b) * a.seq + (qrow < a.seq ? qrow : 0)) * a.emdim + e0;
            for (int c = 0; c < (n_c >> 4); ++c) {
                uint32_t o[16];
                if (t_b > 0) {
                    tmem_ld16(tmem_O + lane_off + c * 16, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = 0u;
                }
                if (qrow < a.seq) {
                    float f[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(o[i]);
                    if (a.bias_o != nullptr) {
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            const uint4 bq =
                                __ldg(reinterpret_cast<const uint4*>(a.bias_o + e0 + c * 16 + g * 8));
                            const __half2* bh = reinterpret_cast<const __half2*>(&bq);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 bf = __half22float2(bh[i]);
                                f[g * 8 + 2 * i] += bf.x;
                                f[g * 8 + 2 * i + 1] += bf.y;
                            }
                        }
                    }
                    uint4 w0, w1;
                    w0.x = pack_half2(f[0], f[1]);
                    w0.y = pack_half2(f[2], f[3]);
                    w0.z = pack_half2(f[4], f[5]);
                    w0.w = pack_half2(f[6], f[7]);
                    w1.x = pack_half2(f[8], f[9]);
                    w1.y = pack_half2(f[10], f[11]);
                    w1.z = pack_half2(f[12], f[13]);
                    w1.w = pack_half2(f[14], f[15]);
                    *reinterpret_cast<uint4*>(orow + c * 16) = w0;
                    *reinterpret_cast<uint4*>(orow + c * 16 + 8) = w1;
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, vo_tmem_cols(NC));
}

}  // namespace
}  // namespace et

namespace et {

int g_vo_chunk = 0;  // test hook: 64 / 128 / 256 output features per CTA, 0 = automatic

// out[t, c] = bias[c] (0 without a bias) for every element.
__global__ void vo_fill_bias_kernel(__half* __restrict__ out, const __half* __restrict__ bias, int T,
                                    int emdim) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = static_cast<size_t>(T) * emdim;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        out[i] = bias ? __ldg(bias + i % emdim) : __float2half_rn(0.f);
}

// out[t, col_id[k]] = comp[t, k] + bias[col_id[k]]: the kept features of a column-pruned result.
__global__ void vo_scatter_cols_kernel(const __half* __restrict__ comp, const int* __restrict__ col_id,
                                       const __half* __restrict__ bias, __half* __restrict__ out,
                                       int T, int nnz_col, int emdim) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = static_cast<size_t>(T) * nnz_col;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = i / nnz_col;
        const int c = __ldg(col_id + (i - t * nnz_col));
        if (c < 0 || c >= emdim) continue;
        const float b = bias ? __half2float(__ldg(bias + c)) : 0.f;
        out[t * emdim + c] = __float2half_rn(__half2float(__ldcg(comp + i)) + b);
    }
}

}  // namespace et

extern "C" {

int et_fused_vo_attention_fwd(const et_half* Q, const et_half* K, const et_half* VO,
                              const et_half* bias_o, et_half* out, int batch, int seq, int nhead,
                              int dh_qk, int emdim, int ldq, int ldk, int mask_kind,
                              const et_half* mask, const int32_t* valid_len, float scale,
                              et_stream stream) {
    using namespace et;
    if (!Q || !K || !VO || !out || batch <= 0 || seq <= 0 || nhead <= 0 || dh_qk <= 0 || emdim <= 0)
        return ET_ERR_INVALID_ARG;
    if (mask_kind < ET_MASK_NONE || mask_kind > ET_MASK_ADDITIVE) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_ADDITIVE && !mask) return ET_ERR_INVALID_ARG;
    if (mask_kind == ET_MASK_PADDING && !valid_len) return ET_ERR_INVALID_ARG;
    if (dh_qk % 16 || dh_qk > 128 || emdim % 16) return ET_ERR_SHAPE;
    if (ldq % 8 || ldk % 8 || ldq < nhead * dh_qk || ldk < nhead * dh_qk) return ET_ERR_SHAPE;
    if (batch > 65535 || static_cast<long>(batch) * nhead > 0x7fffffffL) return ET_ERR_SHAPE;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(VO) || !aligned16(out) ||
        (bias_o && !aligned16(bias_o)))
        return ET_ERR_ALIGNMENT;
    int* err = device_error_word();
    if (!err) return ET_ERR_NO_DEVICE;

    CUtensorMap tmQ, tmK, tmVO;
    const uint32_t box[3] = {64, 128, 1};
    auto make = [&](CUtensorMap* m, const void* p, int ld, int width, int groups) {
        const uint64_t dims[3] = {static_cast<uint64_t>(width), static_cast<uint64_t>(seq),
                                  static_cast<uint64_t>(groups)};
        const uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2,
                                     static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(seq)};
        return make_tensor_map_f16(m, p, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    };
    int st;
    if ((st = make(&tmQ, Q, ldq, nhead * dh_qk, batch)) != ET_OK) return st;
    if ((st = make(&tmK, K, ldk, nhead * dh_qk, batch)) != ET_OK) return st;
    if ((st = make(&tmVO, VO, emdim, emdim, batch * nhead)) != ET_OK) return st;

    VoArgs a;
    a.out = reinterpret_cast<__half*>(out);
    a.bias_o = reinterpret_cast<const __half*>(bias_o);
    a.mask = reinterpret_cast<const __half*>(mask);
    a.valid_len = valid_len;
    a.batch = batch;
    a.seq = seq;
    a.nhead = nhead;
    a.dh_qk = dh_qk;
    a.emdim = emdim;
    a.mask_kind = mask_kind;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.err_word = err;
    // Measured on B200 (12 heads, 768 features; 256 / 128 / 64 features per CTA): 16 x 128 tokens
    // 188 / 195 / 202 us, 64 x 128 376 / 385 / 603, 4 x 512 762 / 794 / 829, 1 x 4096 6.1 / 6.6 /
    // 12.5 ms, and 181-186 us for a single 128-token sequence whatever the width: a CTA's time is
    // set by its serial walk over the heads (about 15 us per head and key block with one set of
    // buffers), not by how many CTAs there are, so the widest chunk runs unless the test hook
    // asks for another.
    int nc = 256;
    if (g_vo_chunk == 64 || g_vo_chunk == 128) nc = g_vo_chunk;
    const int nqa = (dh_qk + 63) / 64;
    int dev = 0;
    cudaGetDevice(&dev);
    auto go = [&](auto kern, int slot, int width) -> int {
        const int smem_bytes = (2 * nqa + width / 64 + 2) * ATOM_BYTES + 256 + 1024;
        static std::atomic<bool> attr_set[3][64] = {};
        if (dev >= 0 && dev < 64 && !attr_set[slot][dev]) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (2 * 2 + width / 64 + 2) * ATOM_BYTES + 256 + 1024) != cudaSuccess)
                return ET_ERR_CUDA;
            attr_set[slot][dev] = true;
        }
        dim3 grid((seq + BQ - 1) / BQ, (emdim + width - 1) / width, batch);
        return launch_kernel(kern, grid, dim3(VO_THREADS), smem_bytes,
                             static_cast<cudaStream_t>(stream), tmQ, tmK, tmVO, a) == cudaSuccess
                   ? ET_OK
                   : ET_ERR_CUDA;
    };
    if (nc == 64) return go(attention_vo_kernel<64>, 0, 64);
    if (nc == 128) return go(attention_vo_kernel<128>, 1, 128);
    return go(attention_vo_kernel<256>, 2, 256);
}

#ifdef ET_TEST_HOOKS
// Test hook: output features per CTA of the pre-multiplied V.O attention (64 / 128 / 256), 0 = automatic.
void et_debug_set_vo_chunk(int nc) { et::g_vo_chunk = nc; }
#endif  // ET_TEST_HOOKS

// ---- column-pruned V.O (Linear_VO_prune + Fused_prune_Multihead_attention) -----------------
// The pre-multiplied weight keeps only the output features col_id[0 .. nnz_col): VO_c is
// [batch][nhead][seq][nnz_col]; the attention runs at that width and its result is scattered
// back to the full feature dimension (pruned features carry the output bias alone).

int et_linear_vo_pruned_fwd(const et_half* X, const et_half* Wvo_c, const et_half* bias,
                            et_half* VOc, int batch, int seq, int nhead, int emdim, int nnz_col,
                            et_stream stream) {
    if (batch <= 0 || seq <= 0 || nhead <= 0 || emdim <= 0 || nnz_col <= 0) return ET_ERR_INVALID_ARG;
    if (emdim % 16 || nnz_col % 16) return ET_ERR_SHAPE;
    return et::launch_gemm_f16_grouped_kn(
        reinterpret_cast<const __half*>(X), emdim, reinterpret_cast<const __half*>(Wvo_c),
        reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(VOc), batch * seq, nnz_col,
        emdim, nhead, seq, static_cast<cudaStream_t>(stream));
}

int et_fused_vo_attention_pruned_fwd(const et_half* Q, const et_half* K, const et_half* VOc,
                                     const int32_t* col_id, int nnz_col, const et_half* bias_o,
                                     et_half* scratch, et_half* out, int batch, int seq, int nhead,
                                     int dh_qk, int emdim, int ldq, int ldk, int mask_kind,
                                     const et_half* mask, const int32_t* valid_len, float scale,
                                     et_stream stream) {
    if (!col_id || !scratch || !out || nnz_col <= 0 || emdim <= 0) return ET_ERR_INVALID_ARG;
    if (nnz_col % 16 || emdim % 8 || nnz_col > emdim) return ET_ERR_SHAPE;
    if (!et::aligned16(out) || !et::aligned16(scratch) || (bias_o && !et::aligned16(bias_o)))
        return ET_ERR_ALIGNMENT;
    int st = et_fused_vo_attention_fwd(Q, K, VOc, nullptr, scratch, batch, seq, nhead, dh_qk, nnz_col,
                                       ldq, ldk, mask_kind, mask, valid_len, scale, stream);
    if (st != ET_OK) return st;
    const int T = batch * seq;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t total = static_cast<size_t>(T) * emdim;
    const int blocks = static_cast<int>((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
    if (et::launch_kernel(et::vo_fill_bias_kernel, dim3(blocks), dim3(256), 0, s,
                          reinterpret_cast<__half*>(out), reinterpret_cast<const __half*>(bias_o), T,
                          emdim) != cudaSuccess)
        return ET_ERR_CUDA;
    const size_t totc = static_cast<size_t>(T) * nnz_col;
    const int blocks2 = static_cast<int>((totc + 255) / 256 < 2048 ? (totc + 255) / 256 : 2048);
    return et::launch_kernel(et::vo_scatter_cols_kernel, dim3(blocks2), dim3(256), 0, s,
                             reinterpret_cast<const __half*>(scratch), col_id,
                             reinterpret_cast<const __half*>(bias_o), reinterpret_cast<__half*>(out),
                             T, nnz_col, emdim) == cudaSuccess
               ? ET_OK
               : ET_ERR_CUDA;
}

}  // extern "C"

