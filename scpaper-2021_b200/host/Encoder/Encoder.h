// Post-LN Transformer encoder layer wired like the reference (Encoder/Encoder.h:49-97):
//   a = attn(x, x, x);  y = LN1(a + x);  f = act(linear1(y));  g = linear2(f);  out = LN2(g + y)
// The activation is folded into linear1's epilogue when its weight format supports it,
// otherwise applied as a separate pass like the reference's act<>.  Nothing is printed.
#pragma once
#include <memory>
#include <type_traits>

#include "../Attention/Attention.h"
#include "../Fused_attention/Fused_attention.h"
#include "../LayerNorm/LayerNorm.h"
#include "../Linear/Linear.h"
#include "../Model.h"
#include "../SkipLayerNorm/SkipLayerNorm.h"

template <typename _attn, typename _l1, typename _l2, typename _act_t> struct Encoder_config {
    using attn_config = _attn;
    using linear1_config = _l1;
    using linear2_config = _l2;
    using act_t = _act_t;
};

struct RELU_OP {};
struct GELU_OP {};

namespace GELU {
// tanh-form GELU over n fp16 values (Encoder/Encoder.cu:41-68)
inline void computeGelu(cudaStream_t stream, int n, const half* input, half* output) {
    etChk(et_act_fwd(et_ptr(input), et_ptr(output), (size_t)n, ET_ACT_GELU, stream));
}
}  // namespace GELU

template <typename ACT_OP_t> constexpr int act_code() {
    return std::is_same_v<ACT_OP_t, RELU_OP> ? ET_ACT_RELU : ET_ACT_GELU;
}

// in-place activation pass (Encoder/Encoder.h:27-37)
template <typename ACT_OP_t> void act(half* data, int size, cudaStream_t stream = 0) {
    etChk(et_act_fwd(et_ptr(data), et_ptr(data), (size_t)size, act_code<ACT_OP_t>(), stream));
}

namespace et_host {
template <typename L, typename = void> struct has_forward_act : std::false_type {};
template <typename L>
struct has_forward_act<L, std::void_t<decltype(std::declval<L&>().forward_act(
                              (half*)nullptr, (const half*)nullptr, 0, (cudaStream_t)0))>>
    : std::true_type {};

template <typename ACT, typename L>
void linear_then_act(L& lin, half* out, half* in, size_t n, cudaStream_t s) {
    if constexpr (has_forward_act<L>::value) {
        lin.forward_act(out, in, act_code<ACT>(), s);
    } else {
        lin.forward(out, in, s);
        act<ACT>(out, (int)n, s);
    }
}
// out = SkipLayerNorm(lin(in), skip).  A dense Linear runs with the LayerNorm in its epilogue
// (one kernel) when the library expects that to pay; otherwise through `tmp`.
template <typename L>
void linear_then_skipln(L& lin, const SkipLayerNorm& ln, half* out, half* tmp, half* in,
                        const half* skip, int rows, cudaStream_t s) {
    if constexpr (std::is_same_v<L, Linear<base_mat>>) {
        if (ln.width() == lin.out_size && lin.size == rows &&
            et_linear_skip_layernorm_pays(rows, lin.in_size, lin.out_size)) {
            etChk(et_linear_skip_layernorm_fwd(et_ptr(in), et_ptr(lin.weight.get()),
                                               et_ptr(lin.bias.get()), et_ptr(skip),
                                               et_ptr(ln.gamma()), et_ptr(ln.beta()), et_ptr(out),
                                               rows, lin.in_size, lin.out_size, s));
            return;
        }
    }
    lin.forward(tmp, in, s);
    ln.forward(out, tmp, skip, rows, s);
}
}  // namespace et_host

template <typename _config> class Encoder {
    using config = _config;
    using attn_t = Attention<typename config::attn_config>;
    using linear1_t = Linear<typename config::linear1_config>;
    using linear2_t = Linear<typename config::linear2_config>;
    using ACT_OP_t = typename config::act_t;

    std::unique_ptr<attn_t> attn;
    std::unique_ptr<SkipLayerNorm> LN1, LN2;
    std::unique_ptr<linear1_t> linear1;
    std::unique_ptr<linear2_t> linear2;
    std::shared_ptr<Model_t> model;
    cudaStream_t stream = 0;

  public:
    culib::CUDA_ptr<half> temp_linear;
    culib::CUDA_ptr<half> temp_attn;
    culib::CUDA_ptr<half> temp_LN;

    Encoder(std::unique_ptr<attn_t> _attn, std::unique_ptr<SkipLayerNorm> _LN1,
            std::unique_ptr<SkipLayerNorm> _LN2, std::unique_ptr<linear1_t> _linear1,
            std::unique_ptr<linear2_t> _linear2, std::shared_ptr<Model_t> _model)
        : attn(std::move(_attn)), LN1(std::move(_LN1)), LN2(std::move(_LN2)),
          linear1(std::move(_linear1)), linear2(std::move(_linear2)), model(_model),
          temp_linear((size_t)et_host::rows_of(*_model) * _model->dimFF),
          temp_attn((size_t)et_host::rows_of(*_model) * _model->emdim),
          temp_LN((size_t)et_host::rows_of(*_model) * _model->emdim) {}

    void set_stream(cudaStream_t s) {
        stream = s;
        attn->set_stream(s);
    }
    attn_t& attention() { return *attn; }

    void forward(half* out, half* src) {
        const int rows = et_host::rows_of(*model);
        if constexpr (attn_t::has_separate_output) {
            half* z = attn->forward_heads(src, src, src);
            et_host::linear_then_skipln(attn->output_linear(), *LN1, temp_LN.get(),
                                        temp_attn.get(), z, src, rows, stream);
        } else {
            attn->forward(temp_attn.get(), src, src, src);
            LN1->forward(temp_LN.get(), temp_attn.get(), src, rows, stream);
        }
        et_host::linear_then_act<ACT_OP_t>(*linear1, temp_linear.get(), temp_LN.get(),
                                           (size_t)rows * model->dimFF, stream);
        et_host::linear_then_skipln(*linear2, *LN2, out, temp_attn.get(), temp_linear.get(),
                                    temp_LN.get(), rows, stream);
    }
};

// Encoder built on the pre-multiplied V.O attention (Encoder/Encoder.h:99-139): tile-pruned
// feed-forward layers, GELU.
template <typename _attn_config> class Encoder_fuse {
    using attn_t = FusedAttention<_attn_config>;
    using linear1_t = Linear<tile_mat>;
    using linear2_t = Linear<tile_mat>;

    std::unique_ptr<attn_t> attn;
    std::unique_ptr<SkipLayerNorm> LN1, LN2;
    std::unique_ptr<linear1_t> linear1;
    std::unique_ptr<linear2_t> linear2;
    std::shared_ptr<Model_t> model;
    cudaStream_t stream = 0;

  public:
    culib::CUDA_ptr<half> temp_linear;
    culib::CUDA_ptr<half> temp_attn;
    culib::CUDA_ptr<half> temp_LN;

    Encoder_fuse(std::unique_ptr<attn_t> _attn, std::unique_ptr<SkipLayerNorm> _LN1,
                 std::unique_ptr<SkipLayerNorm> _LN2, std::unique_ptr<linear1_t> _linear1,
                 std::unique_ptr<linear2_t> _linear2, std::shared_ptr<Model_t> _model)
        : attn(std::move(_attn)), LN1(std::move(_LN1)), LN2(std::move(_LN2)),
          linear1(std::move(_linear1)), linear2(std::move(_linear2)), model(_model),
          temp_linear((size_t)et_host::rows_of(*_model) * _model->dimFF),
          temp_attn((size_t)et_host::rows_of(*_model) * _model->emdim),
          temp_LN((size_t)et_host::rows_of(*_model) * _model->emdim) {}

    void forward(half* out, half* src) {
        const int rows = et_host::rows_of(*model);
        attn->forward(temp_attn.get(), src, src, src);
        LN1->forward(temp_LN.get(), temp_attn.get(), src, rows, stream);
        linear1->forward_act(temp_linear.get(), temp_LN.get(), ET_ACT_GELU, stream);
        linear2->forward(temp_attn.get(), temp_linear.get(), stream);
        LN2->forward(out, temp_attn.get(), temp_LN.get(), rows, stream);
    }
};
