// Attention with pre-multiplied value/output projections (Fused_attention/Fused_attention.h:
// 34-118):  out = sum_h softmax(Q_h K_h^T / sqrt(dh) + mask) (X W_VO,h + b_h) + b_O.
// Both reference variants (OTF_fused_attn, NOTF_fused_attn) resolve to one kernel that keeps
// the output accumulator in tensor memory and reduces heads in a fixed order.
#pragma once
#include <cmath>
#include <memory>

#include "../Attention/Attention.h"
#include "Linear_VO.h"

struct OTF_fused_attn {};
struct NOTF_fused_attn {};

template <typename _config> class FusedAttention {
    using ptr_t = culib::CUDA_ptr<half>;
    using config = _config;
    using linearQ_t = Linear<typename config::WQ_t>;
    using linearK_t = Linear<typename config::WK_t>;

    std::unique_ptr<linearQ_t> linearQ;
    std::unique_ptr<linearK_t> linearK;
    std::unique_ptr<Linear_VO> linearVO;
    ptr_t biasO;
    std::unique_ptr<ptr_t> mat_k, mat_q, mat_vo;
    std::shared_ptr<Model_t> model;
    cudaStream_t stream = 0;

  public:
    FusedAttention(std::unique_ptr<linearQ_t> _linearQ, std::unique_ptr<linearK_t> _linearK,
                   std::unique_ptr<Linear_VO> _linearVO, const ptr_t& _biasO,
                   std::shared_ptr<Model_t> _model)
        : linearQ(std::move(_linearQ)), linearK(std::move(_linearK)),
          linearVO(std::move(_linearVO)), biasO(_biasO), model(_model) {
        const size_t rows = et_host::rows_of(*model);
        mat_k = std::make_unique<ptr_t>(rows * model->kdim);
        mat_q = std::make_unique<ptr_t>(rows * model->kdim);
        mat_vo = std::make_unique<ptr_t>(rows * model->nhead * model->emdim);
    }
    void set_stream(cudaStream_t s) { stream = s; }
    void forward(half* out, half* query, half* key, half* value) {
        linearVO->forward(mat_vo->get(), value, stream);
        linearQ->forward(mat_q->get(), query, stream);
        linearK->forward(mat_k->get(), key, stream);
        const int dh = model->kdim / model->nhead;
        const int kind = model->mask_kind == ET_MASK_CAUSAL ? ET_MASK_CAUSAL : ET_MASK_NONE;
        etChk(et_fused_vo_attention_fwd(et_ptr(mat_q->get()), et_ptr(mat_k->get()),
                                        et_ptr(mat_vo->get()), et_ptr(biasO.get()), et_ptr(out),
                                        model->batch, model->seq_len, model->nhead, dh, model->emdim,
                                        model->kdim, model->kdim, kind, nullptr, nullptr,
                                        1.0f / std::sqrt((float)dh), stream));
    }
};
