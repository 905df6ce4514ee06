// VO[h] = X W_VO[h] + b[h] for the pre-multiplied W_VO = W_V W_O, stored fully pre-processed
// as [nhead][emdim(in)][emdim(out)] row-major (Fused_attention/Linear_VO.h:22-59).  Output
// layout [batch][nhead][seq][emdim].  Linear_VO_prune (Linear_VO.h:61-96) keeps only the
// output features weight.col_id of the product: its weight is a col_mat whose cols are
// [nhead * emdim(in), nnz_col] row-major, its bias [nhead][nnz_col], its output
// [batch][nhead][seq][nnz_col].
#pragma once
#include <memory>

#include "../Model.h"
#include "../lib/CUDA_ptr.hpp"
#include "../mat_type/mat_type.h"

template <typename T> constexpr auto div_ceil(const T& x, const T& y) {
    static_assert(std::is_integral<T>::value, "Integral required.");
    return x / y + (x % y != 0);
}

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

class Linear_VO_prune {
    using ptr_t = culib::CUDA_ptr<half>;

  public:
    ptr_t bias;      // [nhead][nnz_col]
    col_mat weight;  // cols [nhead * emdim, nnz_col], col_id = kept output features
    int head_dim = 0;
    std::shared_ptr<Model_t> model;

    Linear_VO_prune(const col_mat& _weight, const ptr_t& _bias, std::shared_ptr<Model_t> _model)
        : bias(_bias), weight(_weight), model(_model) {}
    void forward(half* output, const half* input, cudaStream_t stream = 0) {
        etChk(et_linear_vo_pruned_fwd(et_ptr(input), et_ptr(weight.cols->get()), et_ptr(bias.get()),
                                      et_ptr(output), model->batch, model->seq_len, model->nhead,
                                      model->emdim, (int)weight.col_id->size, stream));
    }
};
