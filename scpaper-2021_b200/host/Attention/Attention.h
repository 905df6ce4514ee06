// Multi-head self-attention operator with the reference's configuration machinery
// (Attention/Attention.h:10-33): Attention_config<WQ, WK, WV, WO, attn_t, isSingleKernel,
// isPara> selects the weight formats of the four projections and the attention variant.
// Every variant tag resolves to the same on-the-fly tensor-core kernel (scores never reach
// HBM); Prune_attn consumes a column-compressed V, OTF_attn_Ofused folds the tile-pruned
// output projection into the same call.
//   out = O( softmax(Q K^T / sqrt(dh) + mask) V ),   Q, K, V = Linear(x)
// The mask defaults to causal like the reference (Attention.h:97-104); Model_t::mask_kind
// and set_mask() / set_valid_len() select the others.
#pragma once
#include <cassert>
#include <cmath>
#include <memory>
#include <type_traits>

#include "../Linear/Linear.h"
#include "../Model.h"

using ptr_t = culib::CUDA_ptr<half>;

template <typename _WQ_t, typename _WK_t, typename _WV_t, typename _WO_t, typename _attn_t,
          bool _isSingleKernel = false, bool _isPara = true,
          typename = typename std::enable_if<!(_isSingleKernel && _isPara)>::type>
struct Attention_config {
    using WQ_t = _WQ_t;
    using WK_t = _WK_t;
    using WV_t = _WV_t;
    using WO_t = _WO_t;
    using attn_t = _attn_t;
    static constexpr bool isPara = _isPara;
    static constexpr bool isSingleKernel = _isSingleKernel;
    using W_t = typename culib::util::type_if<_isSingleKernel, _WQ_t, void>::type;
};

struct OTF_attn {};
struct Norm_attn {};
struct Prune_attn {};
struct OTF_attn_full {};
struct OTF_attn_tile {};
struct OTF_attn_sharedQK {};
struct OTF_attn_full_mixed {};
struct OTF_attn_Ofused {};

namespace et_host {
struct MaskState {
    int kind;
    const half* additive = nullptr;  // device [seq, seq]
    const int* valid_len = nullptr;  // device [batch]
};
inline int rows_of(const Model_t& m) { return m.batch * m.seq_len; }
}  // namespace et_host

// Free-function form (Attention/Attention.h:35-45,144-181) [sic: "atttion"].  mat_qk is
// accepted for signature compatibility and never touched: scores are not materialised.
// A null mask means "use model->mask_kind"; a non-null one is added to the scaled scores.
template <typename _attn_type>
void Multihead_atttion(ptr_t* mat_q, ptr_t* mat_k, ptr_t* mat_v, ptr_t* /*mat_qk*/,
                       const ptr_t* mask, ptr_t* mat_z, std::shared_ptr<Model_t> model,
                       cudaStream_t stream = 0) {
    const int dh_qk = model->kdim / model->nhead, dh_v = model->vdim / model->nhead;
    const int kind = mask ? ET_MASK_ADDITIVE : (model->mask_kind == ET_MASK_ADDITIVE ? ET_MASK_NONE
                                                                                     : model->mask_kind);
    etChk(et_attention_fwd(et_ptr(mat_q->get()), et_ptr(mat_k->get()), et_ptr(mat_v->get()),
                           et_ptr(mat_z->get()), model->batch, model->seq_len, model->nhead, dh_qk,
                           dh_v, model->kdim, model->kdim, model->vdim, model->vdim, kind,
                           mask ? et_ptr(mask->get()) : nullptr, nullptr,
                           1.0f / std::sqrt((float)dh_qk), stream));
}

// Prune_attn: V arrives as a column-compressed activation (col_mat with head_ptr metadata).
template <typename _attn_type>
void Multihead_atttion(ptr_t* mat_q, ptr_t* mat_k, col_mat* mat_v, ptr_t* /*mat_qk*/,
                       const ptr_t* mask, ptr_t* mat_z, std::shared_ptr<Model_t> model,
                       cudaStream_t stream = 0) {
    const int dh_qk = model->kdim / model->nhead, dh_v = model->vdim / model->nhead;
    const int kind = mask ? ET_MASK_ADDITIVE : (model->mask_kind == ET_MASK_ADDITIVE ? ET_MASK_NONE
                                                                                     : model->mask_kind);
    etChk(et_attention_pruned_v_fwd(
        et_ptr(mat_q->get()), et_ptr(mat_k->get()), et_ptr(mat_v->cols->get()),
        mat_v->col_id->get(), mat_v->head_ptr->get(), mat_v->nnz_col, et_ptr(mat_z->get()),
        model->batch, model->seq_len, model->nhead, dh_qk, dh_v, model->kdim, model->kdim,
        model->vdim, kind, mask ? et_ptr(mask->get()) : nullptr, nullptr,
        1.0f / std::sqrt((float)dh_qk), stream));
}

// Attention + tile-pruned output projection in one call (Attention/kernel_fuseO.h:6-9).
inline void Multihead_atttion_fuseO(half* Q, half* K, half* V, half* mask, half* Z, int* row_ptr,
                                    int* row_offset, half* O_data, half* bias,
                                    std::shared_ptr<Model_t> model, half* out, int o_nnz_tiles,
                                    cudaStream_t stream = 0) {
    const int dh_qk = model->kdim / model->nhead, dh_v = model->vdim / model->nhead;
    const int kind = mask ? ET_MASK_ADDITIVE : (model->mask_kind == ET_MASK_ADDITIVE ? ET_MASK_NONE
                                                                                     : model->mask_kind);
    etChk(et_attention_fuse_o_fwd(et_ptr(Q), et_ptr(K), et_ptr(V), et_ptr(mask), et_ptr(Z), row_ptr,
                                  row_offset, et_ptr(O_data), o_nnz_tiles, et_ptr(bias), et_ptr(out),
                                  model->batch, model->seq_len, model->nhead, dh_qk, dh_v,
                                  model->kdim, model->kdim, model->vdim, model->emdim, kind, nullptr,
                                  1.0f / std::sqrt((float)dh_qk), stream));
}

template <typename T> struct __matv_helper { using type = ptr_t; };
template <> struct __matv_helper<Prune_attn> { using type = col_mat; };

// Q / K / V projections on three side streams joined by events (no host synchronisation).
template <bool _enable, int _nstream> struct parallel_t {
    static constexpr auto nstream = _nstream;
    cudaStream_t streams[_nstream] = {0};
    void fork(cudaStream_t) {}
    void join(cudaStream_t) {}
};
template <int _nstream> struct parallel_t<true, _nstream> {
    static constexpr auto nstream = _nstream;
    cudaStream_t streams[_nstream];
    cudaEvent_t start, done[_nstream];
    parallel_t() {
        cudaChk(cudaEventCreateWithFlags(&start, cudaEventDisableTiming));
        for (int i = 0; i < _nstream; i++) {
            cudaChk(cudaStreamCreateWithFlags(&streams[i], cudaStreamNonBlocking));
            cudaChk(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
    }
    ~parallel_t() {
        for (int i = 0; i < _nstream; i++) {
            cudaStreamDestroy(streams[i]);
            cudaEventDestroy(done[i]);
        }
        cudaEventDestroy(start);
    }
    void fork(cudaStream_t main) {
        cudaChk(cudaEventRecord(start, main));
        for (int i = 0; i < _nstream; i++) cudaChk(cudaStreamWaitEvent(streams[i], start, 0));
    }
    void join(cudaStream_t main) {
        for (int i = 0; i < _nstream; i++) {
            cudaChk(cudaEventRecord(done[i], streams[i]));
            cudaChk(cudaStreamWaitEvent(main, done[i], 0));
        }
    }
};

template <typename _config, typename = void> class Attention {};

// ---- three separate projections (Attention/Attention.h:56-142) ---------------------------
template <typename _config>
class Attention<_config, std::enable_if_t<!_config::isSingleKernel>> {
    using config = _config;
    using linearQ_t = Linear<typename config::WQ_t>;
    using linearK_t = Linear<typename config::WK_t>;
    using linearV_t = Linear<typename config::WV_t>;
    using linearO_t = Linear<typename config::WO_t>;
    using mat_v_t = typename __matv_helper<typename config::attn_t>::type;
    parallel_t<config::isPara, 3> para_handles;

    std::unique_ptr<linearQ_t> linearQ;
    std::unique_ptr<linearK_t> linearK;
    std::unique_ptr<linearV_t> linearV;
    std::unique_ptr<linearO_t> linearO;
    std::unique_ptr<ptr_t> mat_k, mat_q, mat_z;
    std::unique_ptr<mat_v_t> mat_v;
    std::shared_ptr<Model_t> model;
    std::unique_ptr<ptr_t> mask;  // additive mask, only when one was set
    cudaStream_t stream = 0;

  public:
    Attention(std::unique_ptr<linearQ_t> _linearQ, std::unique_ptr<linearK_t> _linearK,
              std::unique_ptr<linearV_t> _linearV, std::unique_ptr<linearO_t> _linearO,
              std::shared_ptr<Model_t> _model)
        : linearQ(std::move(_linearQ)), linearK(std::move(_linearK)), linearV(std::move(_linearV)),
          linearO(std::move(_linearO)), model(_model) {
        static_assert(std::is_same_v<typename config::W_t, void>);
        const size_t rows = et_host::rows_of(*model);
        mat_k = std::make_unique<ptr_t>(rows * model->kdim);
        mat_q = std::make_unique<ptr_t>(rows * model->kdim);
        mat_z = std::make_unique<ptr_t>(rows * model->vdim);
        if constexpr (std::is_same_v<typename config::attn_t, Prune_attn>) {
            static_assert(std::is_same_v<decltype(linearV->weight), row_mat>);
            const int nn = (int)linearV->weight.row_id->size;
            mat_v = std::make_unique<col_mat>((int)rows, model->vdim, nn);
            mat_v->set_metadata(*linearV->weight.row_id, nn, model->nhead, model->vdim);
        } else {
            mat_v = std::make_unique<ptr_t>(rows * model->vdim);
        }
    }
    void set_stream(cudaStream_t s) { stream = s; }
    // additive [seq, seq] mask (host or device pointer); switches the operator to it
    void set_mask(const half* m) {
        mask = std::make_unique<ptr_t>(m, (size_t)model->seq_len * model->seq_len);
    }
    // the output projection is a separate step (not so for the operator that fuses it)
    static constexpr bool has_separate_output =
        !std::is_same_v<OTF_attn_Ofused, typename config::attn_t>;
    linearO_t& output_linear() { return *linearO; }
    // Everything but the output projection; returns Z [rows, vdim].
    half* forward_heads(half* query, half* key, half* value) {
        static_assert(has_separate_output);
        para_handles.fork(stream);
        cudaStream_t sq = config::isPara ? para_handles.streams[0] : stream;
        cudaStream_t sk = config::isPara ? para_handles.streams[1] : stream;
        cudaStream_t sv = config::isPara ? para_handles.streams[2] : stream;
        linearQ->forward(mat_q->get(), query, sq);
        linearK->forward(mat_k->get(), key, sk);
        linearV->forward(mat_v->get(), value, sv);
        para_handles.join(stream);
        Multihead_atttion<typename config::attn_t>(mat_q.get(), mat_k.get(), mat_v.get(), nullptr,
                                                   mask.get(), mat_z.get(), model, stream);
        return mat_z->get();
    }
    void forward(half* out, half* query, half* key, half* value) {
        para_handles.fork(stream);
        cudaStream_t sq = config::isPara ? para_handles.streams[0] : stream;
        cudaStream_t sk = config::isPara ? para_handles.streams[1] : stream;
        cudaStream_t sv = config::isPara ? para_handles.streams[2] : stream;
        linearQ->forward(mat_q->get(), query, sq);
        linearK->forward(mat_k->get(), key, sk);
        linearV->forward(mat_v->get(), value, sv);
        para_handles.join(stream);
        if constexpr (std::is_same_v<OTF_attn_Ofused, typename config::attn_t>) {
            Multihead_atttion_fuseO(mat_q->get(), mat_k->get(), mat_v->get(),
                                    mask ? mask->get() : nullptr, mat_z->get(),
                                    linearO->weight.row_ptr.get(), linearO->weight.row_offset.get(),
                                    linearO->weight.data.get(), linearO->bias.get(), model, out,
                                    linearO->weight.num_blk, stream);
        } else {
            Multihead_atttion<typename config::attn_t>(mat_q.get(), mat_k.get(), mat_v.get(),
                                                       nullptr, mask.get(), mat_z.get(), model,
                                                       stream);
            linearO->forward(out, mat_z->get(), stream);
        }
    }
};

// ---- one fused Q|K|V projection (Attention/Attention.h:204-266): the form the reference's
// paper-table drivers run ------------------------------------------------------------------
template <typename _config>
class Attention<_config, std::enable_if_t<_config::isSingleKernel>> {
    using config = _config;
    using linearQKV_t = Linear<typename config::W_t>;
    using linearO_t = Linear<typename config::WO_t>;

    std::unique_ptr<linearQKV_t> linearQKV;
    std::unique_ptr<linearO_t> linearO;
    std::unique_ptr<ptr_t> mat_qkv, mat_z;
    std::shared_ptr<Model_t> model;
    std::unique_ptr<ptr_t> mask;
    const int* valid_len = nullptr;
    cudaStream_t stream = 0;

  public:
    Attention(std::unique_ptr<linearQKV_t> _linearQKV, std::unique_ptr<linearO_t> _linearO,
              std::shared_ptr<Model_t> _model)
        : linearQKV(std::move(_linearQKV)), linearO(std::move(_linearO)), model(_model) {
        static_assert(!std::is_same_v<typename config::W_t, void>);
        const size_t rows = et_host::rows_of(*model);
        mat_qkv = std::make_unique<ptr_t>(rows * (model->kdim * 2 + model->vdim));
        mat_z = std::make_unique<ptr_t>(rows * model->vdim);
    }
    void set_stream(cudaStream_t s) { stream = s; }
    void set_mask(const half* m) {
        mask = std::make_unique<ptr_t>(m, (size_t)model->seq_len * model->seq_len);
    }
    void set_valid_len(const int* device_lengths) { valid_len = device_lengths; }
    static constexpr bool has_separate_output = true;
    linearO_t& output_linear() { return *linearO; }
    void forward(half* out, half* query, half* key, half* value) {
        linearO->forward(out, forward_heads(query, key, value), stream);
    }
    // Everything but the output projection; returns Z [rows, vdim].
    half* forward_heads(half* query, half* key, half* value) {
        assert(query == key && key == value);
        (void)key;
        (void)value;
        const int ld = model->kdim * 2 + model->vdim;
        const int dh_qk = model->kdim / model->nhead, dh_v = model->vdim / model->nhead;
        int kind = mask ? ET_MASK_ADDITIVE : model->mask_kind;
        if (kind == ET_MASK_ADDITIVE && !mask) kind = ET_MASK_NONE;
        if (kind == ET_MASK_PADDING && !valid_len) kind = ET_MASK_NONE;
        if constexpr (std::is_same_v<typename config::W_t, base_mat>) {
            // dense fused-QKV weight, short sequences, 64-wide heads: projection and attention
            // run as one kernel and the projected activations never reach memory
            if (model->seq_len <= 128 && dh_qk == 64 && dh_v == 64) {
                etChk(et_qkv_attention_fwd(et_ptr(query), et_ptr(linearQKV->weight.get()),
                                           et_ptr(linearQKV->bias.get()), et_ptr(mat_z->get()),
                                           model->batch, model->seq_len, linearQKV->in_size,
                                           model->nhead, model->kdim, model->vdim, kind,
                                           mask ? et_ptr(mask->get()) : nullptr, valid_len,
                                           1.0f / std::sqrt((float)dh_qk), stream));
                return mat_z->get();
            }
        }
        linearQKV->forward(mat_qkv->get(), query, stream);
        half* Q = mat_qkv->get();
        half* K = Q + model->kdim;
        half* V = K + model->kdim;
        etChk(et_attention_fwd(et_ptr(Q), et_ptr(K), et_ptr(V), et_ptr(mat_z->get()), model->batch,
                               model->seq_len, model->nhead, dh_qk, dh_v, ld, ld, ld, model->vdim,
                               kind, mask ? et_ptr(mask->get()) : nullptr, valid_len,
                               1.0f / std::sqrt((float)dh_qk), stream));
        return mat_z->get();
    }
};
