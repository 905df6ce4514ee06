// out = LayerNorm(src + skip) * weight + bias, eps 1e-5, one row per token
// (SkipLayerNorm/SkipLayerNorm.h:6-18).  Statistics are fp32 and the variance is
// E[x^2] - E[x]^2 (the reference kernel subtracts the unsquared mean).
#pragma once
#include <memory>

#include "../lib/CUDA_ptr.hpp"

class SkipLayerNorm {
    const int size;
    culib::CUDA_ptr<half> weight;
    culib::CUDA_ptr<half> bias;

  public:
    SkipLayerNorm(const half* w, const half* b, int _size)
        : size(_size), weight(w, _size), bias(b, _size) {}
    int width() const { return size; }
    const half* gamma() const { return weight.get(); }
    const half* beta() const { return bias.get(); }
    void forward(half* out, const half* src, const half* skip, int num,
                 cudaStream_t stream = 0) const {
        etChk(et_skip_layernorm_fwd(et_ptr(src), et_ptr(skip), et_ptr(weight.get()),
                                    et_ptr(bias.get()), et_ptr(out), num, size, stream));
    }
};

// weight = bias = 0.2 like the reference generator (SkipLayerNorm.cu:84-89)
inline std::unique_ptr<SkipLayerNorm> gen_skLN(int size) {
    std::vector<half> v(size, __float2half_rn(0.2f));
    return std::make_unique<SkipLayerNorm>(v.data(), v.data(), size);
}
