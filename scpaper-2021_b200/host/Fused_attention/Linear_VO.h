// VO[h] = X W_VO[h] + b[h] for the pre-multiplied W_VO = W_V W_O, stored fully pre-processed
// as [nhead][emdim(in)][emdim(out)] row-major (Fused_attention/Linear_VO.h:22-59).  Output
// layout [batch][nhead][seq][emdim].
#pragma once
#include <memory>

#include "../Model.h"
#include "../lib/CUDA_ptr.hpp"

class Linear_VO {
    using ptr_t = culib::CUDA_ptr<half>;

  public:
    ptr_t bias;    // [nhead][emdim]
    ptr_t weight;  // [nhead][emdim][emdim]
    std::shared_ptr<Model_t> model;

    Linear_VO(const ptr_t& _weight, const ptr_t& _bias, std::shared_ptr<Model_t> _model)
        : bias(_bias), weight(_weight), model(_model) {}
    void forward(half* output, const half* input, cudaStream_t stream = 0) {
        etChk(et_linear_vo_fwd(et_ptr(input), et_ptr(weight.get()), et_ptr(bias.get()),
                               et_ptr(output), model->batch, model->seq_len, model->nhead,
                               model->emdim, stream));
    }
};
