// Attention with pre-multiplied value/output projections (Fused_attention/Fused_attention.h:
// 12-130):  out = sum_h softmax(Q_h K_h^T / sqrt(dh) + mask) (X W_VO,h + b_h) + b_O.
// The reference's variants (OTF_fused_attn with half2 atomics across heads, NOTF_fused_attn
// with the probabilities written to memory and one big GEMM) resolve to one kernel that keeps
// the output accumulator in tensor memory and reduces heads in a fixed order;
// NOTF_fused_prune_attn runs it at the width of the kept output features and scatters.
//
// Free functions keep the reference's parameter lists.  mat_qk, the cuBLAS handle and the
// V.O stream are accepted and ignored (scores are never materialised, no cuBLAS call is made,
// everything is ordered on one stream).  A non-null mask is an additive [seq, seq] fp16 mask;
// a null mask selects model->mask_kind (additive falls back to none).  Like the reference's,
// the free functions do not add the output bias.
#pragma once
#include <cublas_v2.h>

#include <cmath>
#include <memory>
#include <type_traits>

#include "../Attention/Attention.h"
#include "../lib/cuda_map.cuh"
#include "Linear_VO.h"

struct OTF_fused_attn {};
struct NOTF_fused_attn {};
struct NOTF_fused_prune_attn {};

namespace et_host {
inline int fused_mask_kind(const culib::CUDA_ptr<half>* mask, const Model_t& m, const int* valid_len) {
    if (mask) return ET_MASK_ADDITIVE;
    if (m.mask_kind == ET_MASK_ADDITIVE) return ET_MASK_NONE;
    if (m.mask_kind == ET_MASK_PADDING && !valid_len) return ET_MASK_NONE;
    return m.mask_kind;
}
inline void fused_vo_attention(half* mat_q, half* mat_k, half* mat_vo,
                               const culib::CUDA_ptr<half>* mask, const int* valid_len,
                               const half* bias_o, half* output, const Model_t& m,
                               cudaStream_t stream) {
    const int dh = m.kdim / m.nhead;
    etChk(et_fused_vo_attention_fwd(et_ptr(mat_q), et_ptr(mat_k), et_ptr(mat_vo), et_ptr(bias_o),
                                    et_ptr(output), m.batch, m.seq_len, m.nhead, dh, m.emdim, m.kdim,
                                    m.kdim, fused_mask_kind(mask, m, valid_len),
                                    mask ? et_ptr(mask->get()) : nullptr, valid_len,
                                    1.0f / std::sqrt((float)dh), stream));
}
inline void fused_vo_attention_pruned(half* mat_q, half* mat_k, half* mat_vo,
                                      const culib::CUDA_ptr<half>* mask, const int* valid_len,
                                      const half* bias_o, half* output, half* mat_vos,
                                      const Model_t& m, Linear_VO_prune* linearVO,
                                      cudaStream_t stream) {
    const int dh = m.kdim / m.nhead;
    etChk(et_fused_vo_attention_pruned_fwd(
        et_ptr(mat_q), et_ptr(mat_k), et_ptr(mat_vo), linearVO->weight.col_id->get(),
        (int)linearVO->weight.col_id->size, et_ptr(bias_o), et_ptr(mat_vos), et_ptr(output), m.batch,
        m.seq_len, m.nhead, dh, m.emdim, m.kdim, m.kdim, fused_mask_kind(mask, m, valid_len),
        mask ? et_ptr(mask->get()) : nullptr, valid_len, 1.0f / std::sqrt((float)dh), stream));
}
}  // namespace et_host

// Fused_attention.h:12-18 and its two specialisations (:119-130).
template <typename attn_t>
void Fused_Multihead_attention(half* mat_q, half* mat_k, half* mat_vo, half* /*mat_qk*/,
                               const culib::CUDA_ptr<half>* mask, half* output,
                               std::shared_ptr<Model_t> model, cublasHandle_t /*handle*/,
                               cudaStream_t streamVO) {
    static_assert(std::is_same_v<attn_t, OTF_fused_attn> || std::is_same_v<attn_t, NOTF_fused_attn>,
                  "Unknown attention");
    et_host::fused_vo_attention(mat_q, mat_k, mat_vo, mask, nullptr, nullptr, output, *model,
                                streamVO);
}

// Fused_attention.h:19-23 (Fused_attention.cu:273-309): mat_vos is scratch [rows, nnz_col].
inline void Fused_prune_Multihead_attention(half* mat_q, half* mat_k, half* mat_vo, half* /*mat_qk*/,
                                            const culib::CUDA_ptr<half>* mask, half* output,
                                            half* mat_vos, std::shared_ptr<Model_t> model,
                                            cublasHandle_t /*handle*/, Linear_VO_prune* linearVO,
                                            cudaStream_t streamVO) {
    et_host::fused_vo_attention_pruned(mat_q, mat_k, mat_vo, mask, nullptr, nullptr, output, mat_vos,
                                       *model, linearVO, streamVO);
}

template <typename T> struct __VO_helper { using type = Linear_VO; };
template <> struct __VO_helper<NOTF_fused_prune_attn> { using type = Linear_VO_prune; };

template <typename _config> class FusedAttention {
    using ptr_t = culib::CUDA_ptr<half>;
    using config = _config;
    using linearQ_t = Linear<typename config::WQ_t>;
    using linearK_t = Linear<typename config::WK_t>;
    using LinearVO_t = typename __VO_helper<typename config::attn_t>::type;
    static constexpr bool pruned = std::is_same_v<typename config::attn_t, NOTF_fused_prune_attn>;

    std::unique_ptr<linearQ_t> linearQ;
    std::unique_ptr<linearK_t> linearK;
    std::unique_ptr<LinearVO_t> linearVO;
    ptr_t biasO;
    std::unique_ptr<ptr_t> mat_k, mat_q, mat_vo, mat_vos;
    std::shared_ptr<Model_t> model;
    std::unique_ptr<ptr_t> mask;  // additive mask, only when one was set
    const int* valid_len = nullptr;
    cudaStream_t stream = 0;

  public:
    FusedAttention(std::unique_ptr<linearQ_t> _linearQ, std::unique_ptr<linearK_t> _linearK,
                   std::unique_ptr<LinearVO_t> _linearVO, const ptr_t& _biasO,
                   std::shared_ptr<Model_t> _model)
        : linearQ(std::move(_linearQ)), linearK(std::move(_linearK)),
          linearVO(std::move(_linearVO)), biasO(_biasO), model(_model) {
        const size_t rows = et_host::rows_of(*model);
        mat_k = std::make_unique<ptr_t>(rows * model->kdim);
        mat_q = std::make_unique<ptr_t>(rows * model->kdim);
        if constexpr (pruned) {
            const size_t nnz = linearVO->weight.col_id->size;
            mat_vo = std::make_unique<ptr_t>(rows * model->nhead * nnz);
            mat_vos = std::make_unique<ptr_t>(rows * nnz);
        } else {
            mat_vo = std::make_unique<ptr_t>(rows * model->nhead * model->emdim);
        }
    }
    void set_stream(cudaStream_t s) { stream = s; }
    // additive [seq, seq] mask (host or device pointer); switches the operator to it
    void set_mask(const half* m) {
        mask = std::make_unique<ptr_t>(m, (size_t)model->seq_len * model->seq_len);
    }
    // per-sequence key counts (device, [batch]) for Model_t::mask_kind == ET_MASK_PADDING
    void set_valid_len(const int* device_lengths) { valid_len = device_lengths; }
    void forward(half* out, half* query, half* key, half* value) {
        linearVO->forward(mat_vo->get(), value, stream);
        linearQ->forward(mat_q->get(), query, stream);
        linearK->forward(mat_k->get(), key, stream);
        if constexpr (pruned)
            et_host::fused_vo_attention_pruned(mat_q->get(), mat_k->get(), mat_vo->get(), mask.get(),
                                               valid_len, biasO.get(), out, mat_vos->get(), *model,
                                               linearVO.get(), stream);
        else
            et_host::fused_vo_attention(mat_q->get(), mat_k->get(), mat_vo->get(), mask.get(),
                                        valid_len, biasO.get(), out, *model, stream);
    }
};
