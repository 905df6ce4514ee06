// Whole post-LN encoder layer: the sequence of launches Encoder<config>::forward makes in
// the reference (Encoder/Encoder.h:81-96), with bias / activation folded into the GEMM
// epilogues and the fused [Q | K | V] projection feeding the on-the-fly attention kernel.
//
//   qkv = QKV(x)                      [T, 2*kdim + vdim]
//   z   = attention(qkv)              [T, vdim]
//   a   = O(z)                        [T, hidden]
//   y   = LN1(a + x)                  [T, hidden]
//   f   = act(W1 y + b1)              [T, ff]
//   a   = W2 f + b2                   [T, hidden]
//   out = LN2(a + y)
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace et {
namespace {

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

constexpr int kMaxSplits = 4;

struct LayerBuffers {
    __half *qkv, *z, *a, *y, *f;
    __half* gather;  // [T, widest column-pruned input]: scratch of the column-pruned Linears
    size_t gather_bytes;
    float* part;  // split-K partial sums [kMaxSplits][T, hidden]
    size_t total;
};

// A row-pruned FFN1 feeding a column-pruned FFN2 over the same id list: the pruned hidden
// units of the feed-forward block.  Both products then run at the kept width.
bool ffn_is_compressed_pair(const et_encoder_layer_t* L) {
    return L->ffn1.format == ET_FMT_ROW && L->ffn2.format == ET_FMT_COL &&
           L->ffn1.row_ptr != nullptr && L->ffn1.row_ptr == L->ffn2.row_ptr &&
           L->ffn1.nnz_tiles == L->ffn2.nnz_tiles && L->ffn1.nnz_tiles > 0 &&
           L->ffn1.nnz_tiles % 8 == 0;
}

// Number of K slices for a dense [T, K] x [hidden, K]^T product feeding a LayerNorm: few
// output tiles and a long K leave most SMs idle unless K is split.
int g_force_splits = 0;  // test hook: 0 = automatic
bool g_qkv_fusion = true;  // test hook: false = always the separate projection + attention
// test hook: which dense Linear + skip-LayerNorm pairs run as one kernel (gemm_ln.cu):
// -1 = automatic, otherwise a mask: 1 = the O projection, 2 = FFN2
int g_ln_fusion = -1;

// The fused kernel computes 128 x 128 tiles, one per CTA, in clusters of hidden / 128 CTAs.
// Measured on B200: while all its clusters are resident at once it beats the separate GEMM +
// LayerNorm (BERT-base, 2048 tokens: 8.0 vs 10.8 us for the O projection, 15.3 vs 18.4 us for
// FFN2, +10 % on the whole stack); with several waves the wider tiles and CTA pairs of the plain
// GEMM win by more than the LayerNorm launch costs (8192 tokens: -3 %).  A cluster must fit one
// GPC, so the number of resident clusters comes from the occupancy query, not from the SM count.
int ln_fusion_mask(int T, int hidden) {
    if (g_ln_fusion >= 0) return g_ln_fusion;
    return et_linear_skip_layernorm_pays(T, hidden, hidden) ? 3 : 0;
}

// Split-K on CTA pairs: 256 x 256 pair tiles, as many K slices as SM pairs allow.  Returns 0
// when the pair form does not apply.  Measured on B200 at BERT-base sizes the fp32 partial
// sums (written by the GEMM, re-read by the LayerNorm) cost more than the better machine fill
// gains, so this form only runs when the test hook asks for it (-2).
int pick_pair_splits(int T, int hidden, int K) {
    if (g_force_splits != -2) return 0;
    if (T < 256 || hidden < 256) return 0;
    const int pairs = (sm_count() > 0 ? sm_count() : 148) / 2;
    const int tiles = ((T + 255) / 256) * ((hidden + 255) / 256);
    int s = pairs / tiles;
    s = s > kMaxSplits ? kMaxSplits : s;
    while (s > 1 && (K / 64) / s < 8) --s;  // keep at least 8 K blocks per slice
    return s >= 2 ? s : 0;
}

int pick_splits(int T, int hidden, int K) {
    if (g_force_splits > 0) return g_force_splits > kMaxSplits ? kMaxSplits : g_force_splits;
    const int tiles = ((T + 127) / 128) * ((hidden + 127) / 128);
    const int slots = 2 * (sm_count() > 0 ? sm_count() : 148);
    int s = slots / (tiles > 0 ? tiles : 1);
    s = s < 1 ? 1 : (s > kMaxSplits ? kMaxSplits : s);
    while (s > 1 && (K / 64) / s < 8) --s;  // keep at least 8 K blocks per slice
    // With persistent CTAs a half-filled machine already overlaps its epilogues; the extra
    // fp32 traffic of the partial sums only pays when very few tiles exist.
    if (2 * tiles > (sm_count() > 0 ? sm_count() : 148)) s = 1;
    return s;
}

LayerBuffers carve(const et_encoder_layer_t* L, int batch, int seq, void* base) {
    const size_t T = static_cast<size_t>(batch) * seq;
    LayerBuffers b;
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    auto take = [&](size_t elems) {
        __half* r = reinterpret_cast<__half*>(p + off);
        off += align256(elems * sizeof(__half));
        return r;
    };
    b.qkv = take(T * (2 * static_cast<size_t>(L->kdim) + L->vdim));
    b.z = take(T * L->vdim);
    b.a = take(T * L->hidden);
    b.y = take(T * L->hidden);
    b.f = take(T * L->ff);
    size_t widest = 0;
    for (const et_linear_t* lin : {&L->qkv, &L->o, &L->ffn1, &L->ffn2})
        if (lin->format == ET_FMT_COL && lin->nnz_tiles > 0 &&
            static_cast<size_t>(lin->nnz_tiles) > widest)
            widest = static_cast<size_t>(lin->nnz_tiles);
    if (ffn_is_compressed_pair(L)) widest = 0;  // that pair needs no gather
    b.gather_bytes = T * widest * sizeof(__half);
    b.gather = take(T * widest);
    b.part = reinterpret_cast<float*>(take(2 * kMaxSplits * T * L->hidden));
    b.total = off;
    return b;
}

int run_linear(const et_linear_t& lin, const __half* X, __half* Y, int T, int act,
               const LayerBuffers& buf, cudaStream_t stream) {
    const et_half* Xe = reinterpret_cast<const et_half*>(X);
    et_half* Ye = reinterpret_cast<et_half*>(Y);
    switch (lin.format) {
        case ET_FMT_1X16:
            return et_linear_1x16_fwd(lin.row_ptr, lin.row_off, lin.weight, lin.nnz_tiles, lin.bias,
                                      Xe, Ye, T, lin.in, lin.out, act, stream);
        case ET_FMT_ROW:
            return et_linear_row_fwd(lin.row_ptr, lin.weight, lin.nnz_tiles, lin.bias, Xe, Ye, T,
                                     lin.in, lin.out, act, stream);
        case ET_FMT_COL:
            return et_linear_col_fwd(lin.row_ptr, lin.weight, lin.nnz_tiles, lin.bias, Xe, Ye, T,
                                     lin.in, lin.out, act, reinterpret_cast<et_half*>(buf.gather),
                                     buf.gather_bytes, stream);
        case ET_FMT_CSR:
            return et_linear_csr_fwd(lin.row_ptr, lin.row_off, lin.weight, lin.nnz_tiles, lin.bias,
                                     Xe, Ye, T, lin.in, lin.out, act, stream);
        default: break;
    }
    if (lin.format == ET_FMT_DENSE)
        return launch_gemm_f16(X, lin.in, reinterpret_cast<const __half*>(lin.weight), lin.in,
                               reinterpret_cast<const __half*>(lin.bias), Y, lin.out, nullptr, 0, T,
                               lin.out, lin.in, act, stream);
    if (lin.format == ET_FMT_TILE)
        return launch_linear_tile(lin.row_ptr, lin.row_off,
                                  reinterpret_cast<const __half*>(lin.weight), lin.nnz_tiles,
                                  reinterpret_cast<const __half*>(lin.bias), X, Y, T, lin.in,
                                  lin.out, act, stream);
    if (lin.format == ET_FMT_TILE_PACKED)
        return launch_linear_tile_packed(lin.row_ptr, lin.pk_mask, lin.pk_off,
                                         reinterpret_cast<const __half*>(lin.weight), lin.nnz_tiles,
                                         reinterpret_cast<const __half*>(lin.bias), X, Y, T, lin.in,
                                         lin.out, act, stream);
    return ET_ERR_INVALID_ARG;
}

int check_layer(const et_encoder_layer_t* L) {
    if (!L) return ET_ERR_INVALID_ARG;
    if (L->hidden <= 0 || L->nhead <= 0 || L->kdim <= 0 || L->vdim <= 0 || L->ff <= 0)
        return ET_ERR_INVALID_ARG;
    if (L->kdim % L->nhead || L->vdim % L->nhead) return ET_ERR_SHAPE;
    if (L->qkv.in != L->hidden || L->qkv.out != 2 * L->kdim + L->vdim) return ET_ERR_SHAPE;
    if (L->o.in != L->vdim || L->o.out != L->hidden) return ET_ERR_SHAPE;
    if (L->ffn1.in != L->hidden || L->ffn1.out != L->ff) return ET_ERR_SHAPE;
    if (L->ffn2.in != L->ff || L->ffn2.out != L->hidden) return ET_ERR_SHAPE;
    if (!L->ln1_gamma || !L->ln1_beta || !L->ln2_gamma || !L->ln2_beta) return ET_ERR_INVALID_ARG;
    if (L->act != ET_ACT_RELU && L->act != ET_ACT_GELU) return ET_ERR_INVALID_ARG;
    return ET_OK;
}


// y = b.y (the first LayerNorm's output) -> out = LN2(W2 act(W1 y + b1) + b2 + y)
int ffn_block(const et_encoder_layer_t* layer, const LayerBuffers& b, int T, __half* out_h,
              cudaStream_t s) {
    int st;
    et_half* out = reinterpret_cast<et_half*>(out_h);
    const int ln_fused = ln_fusion_mask(T, layer->hidden);
    // ffn2 as the dense product it amounts to: W2 itself, or - for the compressed pair - the
    // kept columns of W2 on the kept hidden units
    const __half* w2 = reinterpret_cast<const __half*>(layer->ffn2.weight);
    int k2 = layer->ff;
    bool ffn2_dense = layer->ffn2.format == ET_FMT_DENSE;
    if (ffn_is_compressed_pair(layer)) {
        k2 = layer->ffn1.nnz_tiles;
        ffn2_dense = true;
        // f[T, kept] = act(y . rows^T + b1[kept ids]): GEMM with an index-list epilogue
        if ((st = launch_gemm_f16(b.y, layer->hidden,
                                      reinterpret_cast<const __half*>(layer->ffn1.weight),
                                      layer->hidden,
                                      reinterpret_cast<const __half*>(layer->ffn1.bias), b.f, k2,
                                      layer->ffn1.row_ptr, 0, T, k2, layer->hidden, layer->act,
                                      s)) != ET_OK)
            return st;
    } else if ((st = run_linear(layer->ffn1, b.y, b.f, T, layer->act, b, s)) != ET_OK) {
        return st;
    }
    if ((ln_fused & 2) && ffn2_dense && gemm_ln_applies(T, layer->hidden, k2) &&
        reinterpret_cast<const __half*>(out) != b.y) {
        // FFN2, residual and LayerNorm in one kernel
        return launch_gemm_ln(b.f, k2, w2, k2,
                                  reinterpret_cast<const __half*>(layer->ffn2.bias), b.y,
                                  layer->hidden,
                                  reinterpret_cast<const __half*>(layer->ln2_gamma),
                                  reinterpret_cast<const __half*>(layer->ln2_beta),
                                  reinterpret_cast<__half*>(out), layer->hidden, T, layer->hidden,
                                  k2, s);
    }
    const bool ffn2_splittable = ffn2_dense && layer->hidden <= 2048;
    const int pair_splits =
        ffn2_splittable ? pick_pair_splits(T, layer->hidden, k2) : 0;
    if (pair_splits > 1) {
        // FFN2 as split-K partial sums on CTA pairs, reduced (with bias and residual) inside
        // the LayerNorm
        if ((st = launch_gemm_pair_splitk(b.f, k2, w2, k2, b.part, T, layer->hidden, k2,
                                              pair_splits, s)) != ET_OK)
            return st;
        return launch_skip_layernorm_partials(
            b.part, pair_splits, static_cast<size_t>(T) * layer->hidden,
            reinterpret_cast<const __half*>(layer->ffn2.bias), b.y,
            reinterpret_cast<const __half*>(layer->ln2_gamma),
            reinterpret_cast<const __half*>(layer->ln2_beta), reinterpret_cast<__half*>(out), T,
            layer->hidden, s);
    }
    const int splits = ffn2_splittable ? pick_splits(T, layer->hidden, k2) : 1;
    if (splits > 1) {
        // FFN2 as split-K partial sums, reduced (with bias and residual) inside the LayerNorm
        if ((st = launch_gemm_f16_splitk(b.f, k2, w2, k2, b.part, T, layer->hidden, k2, splits,
                                             s)) != ET_OK)
            return st;
        return launch_skip_layernorm_partials(
            b.part, splits, static_cast<size_t>(T) * layer->hidden,
            reinterpret_cast<const __half*>(layer->ffn2.bias), b.y,
            reinterpret_cast<const __half*>(layer->ln2_gamma),
            reinterpret_cast<const __half*>(layer->ln2_beta), reinterpret_cast<__half*>(out), T,
            layer->hidden, s);
    }
    if (ffn2_dense && layer->ffn2.format != ET_FMT_DENSE) {
        if ((st = launch_gemm_f16(b.f, k2, w2, k2,
                                      reinterpret_cast<const __half*>(layer->ffn2.bias), b.a,
                                      layer->hidden, nullptr, 0, T, layer->hidden, k2, ET_ACT_NONE,
                                      s)) != ET_OK)
            return st;
    } else if ((st = run_linear(layer->ffn2, b.f, b.a, T, ET_ACT_NONE, b, s)) != ET_OK) {
        return st;
    }
    return launch_skip_layernorm(b.a, b.y, reinterpret_cast<const __half*>(layer->ln2_gamma),
                                     reinterpret_cast<const __half*>(layer->ln2_beta),
                                     reinterpret_cast<__half*>(out), T, layer->hidden, s);
}

}  // namespace
}  // namespace et

extern "C" {

#ifdef ET_TEST_HOOKS
// Test hook: number of K slices of the FFN2 product (0 = automatic, 1 = no split, n > 1 = n
// slices on single-CTA tiles, -2 = K slices on 256 x 256 CTA-pair tiles).
void et_debug_force_ffn2_splits(int n) { et::g_force_splits = n; }

// Test hook: 0 = never fuse the Q/K/V projection into the attention kernel.
void et_debug_set_qkv_fusion(int on) { et::g_qkv_fusion = on != 0; }
void et_debug_set_ln_fusion(int mode) { et::g_ln_fusion = mode; }
#endif  // ET_TEST_HOOKS

size_t et_encoder_layer_workspace_bytes(const et_encoder_layer_t* layer, int batch, int seq) {
    if (et::check_layer(layer) != ET_OK || batch <= 0 || seq <= 0) return 0;
    return et::carve(layer, batch, seq, nullptr).total;
}

int et_encoder_layer_fwd(const et_encoder_layer_t* layer, const et_half* x, et_half* out,
                         int batch, int seq, int mask_kind, const et_half* mask,
                         const int32_t* valid_len, void* workspace, size_t workspace_bytes,
                         et_stream stream) {
    int st = et::check_layer(layer);
    if (st != ET_OK) return st;
    if (!x || !out || batch <= 0 || seq <= 0) return ET_ERR_INVALID_ARG;
    if (!workspace) return ET_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return ET_ERR_ALIGNMENT;
    const et::LayerBuffers b = et::carve(layer, batch, seq, workspace);
    if (workspace_bytes < b.total) return ET_ERR_WORKSPACE;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int T = batch * seq;
    const __half* xin = reinterpret_cast<const __half*>(x);
    const int ldqkv = 2 * layer->kdim + layer->vdim;
    const int dh_qk = layer->kdim / layer->nhead, dh_v = layer->vdim / layer->nhead;

    // The fused kernel projects a full 128-token block per sequence whatever its length: below
    // 96 tokens the padding costs more than the fusion saves (measured at 64: 4 % slower).
    if (et::g_qkv_fusion && layer->qkv.format == ET_FMT_DENSE && seq >= 96 &&
        et::qkv_attention_applies(seq, layer->nhead, layer->kdim, layer->vdim)) {
        // short sequences, 64-wide heads: projection and attention in one kernel, the projected
        // Q / K / V never leave the SM
        if ((st = et::launch_qkv_attention(
                 xin, reinterpret_cast<const __half*>(layer->qkv.weight),
                 reinterpret_cast<const __half*>(layer->qkv.bias), b.z, batch, seq, layer->hidden,
                 layer->nhead, layer->kdim, layer->vdim, layer->vdim, mask_kind,
                 reinterpret_cast<const __half*>(mask), valid_len,
                 1.0f / sqrtf(static_cast<float>(dh_qk)), s)) != ET_OK)
            return st;
    } else {
        if ((st = et::run_linear(layer->qkv, xin, b.qkv, T, ET_ACT_NONE, b, s)) != ET_OK) return st;
        if ((st = et::launch_attention(b.qkv, b.qkv + layer->kdim, b.qkv + 2 * layer->kdim, b.z,
                                       batch, seq, layer->nhead, dh_qk, dh_v, ldqkv, ldqkv, ldqkv,
                                       layer->vdim, mask_kind, reinterpret_cast<const __half*>(mask),
                                       valid_len, 1.0f / sqrtf(static_cast<float>(dh_qk)), s)) !=
            ET_OK)
            return st;
    }
    const int ln_fused = et::ln_fusion_mask(T, layer->hidden);
    if ((ln_fused & 1) && layer->o.format == ET_FMT_DENSE &&
        et::gemm_ln_applies(T, layer->hidden, layer->vdim)) {
        // O projection, residual and LayerNorm in one kernel
        if ((st = et::launch_gemm_ln(b.z, layer->vdim,
                                     reinterpret_cast<const __half*>(layer->o.weight), layer->vdim,
                                     reinterpret_cast<const __half*>(layer->o.bias), xin,
                                     layer->hidden,
                                     reinterpret_cast<const __half*>(layer->ln1_gamma),
                                     reinterpret_cast<const __half*>(layer->ln1_beta), b.y,
                                     layer->hidden, T, layer->hidden, layer->vdim, s)) != ET_OK)
            return st;
    } else {
        if ((st = et::run_linear(layer->o, b.z, b.a, T, ET_ACT_NONE, b, s)) != ET_OK) return st;
        if ((st = et::launch_skip_layernorm(b.a, xin,
                                            reinterpret_cast<const __half*>(layer->ln1_gamma),
                                            reinterpret_cast<const __half*>(layer->ln1_beta), b.y,
                                            T, layer->hidden, s)) != ET_OK)
            return st;
    }
    return et::ffn_block(layer, b, T, reinterpret_cast<__half*>(out), s);
}

// ---- head-parallel form: the layer in two halves around the ranks' one exchange step --------
int et_encoder_attention_units_fwd(const et_encoder_layer_t* layer, const et_half* x, void* partial,
                                   int partial_is_f32, int batch, int seq, int mask_kind,
                                   const et_half* mask, const int32_t* valid_len,
                                   const int32_t* unit_head, const int32_t* unit_first_block,
                                   int n_units, int blocks_per_unit, void* workspace,
                                   size_t workspace_bytes, et_stream stream) {
    int st = et::check_layer(layer);
    if (st != ET_OK) return st;
    if (!x || !partial || batch <= 0 || seq <= 0 || n_units <= 0) return ET_ERR_INVALID_ARG;
    if (layer->qkv.format != ET_FMT_DENSE || layer->o.format != ET_FMT_DENSE) return ET_ERR_SHAPE;
    if (!workspace) return ET_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return ET_ERR_ALIGNMENT;
    const et::LayerBuffers b = et::carve(layer, batch, seq, workspace);
    if (workspace_bytes < b.total) return ET_ERR_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int T = batch * seq;
    const int ldqkv = 2 * layer->kdim + layer->vdim;
    const int dh_qk = layer->kdim / layer->nhead, dh_v = layer->vdim / layer->nhead;
    // rows of z outside this rank's units must contribute nothing to the partial product
    if (cudaMemsetAsync(b.z, 0, static_cast<size_t>(T) * layer->vdim * sizeof(__half), s) != cudaSuccess)
        return ET_ERR_CUDA;
    if ((st = et::run_linear(layer->qkv, reinterpret_cast<const __half*>(x), b.qkv, T, ET_ACT_NONE, b,
                             s)) != ET_OK)
        return st;
    if ((st = et::launch_attention_units(b.qkv, b.qkv + layer->kdim, b.qkv + 2 * layer->kdim, b.z,
                                         batch, seq, layer->nhead, dh_qk, dh_v, ldqkv, ldqkv, ldqkv,
                                         layer->vdim, mask_kind, reinterpret_cast<const __half*>(mask),
                                         valid_len, 1.0f / sqrtf(static_cast<float>(dh_qk)), unit_head,
                                         unit_first_block, n_units, blocks_per_unit, s)) != ET_OK)
        return st;
    if (partial_is_f32)
        return et::launch_gemm_f16_splitk(b.z, layer->vdim,
                                          reinterpret_cast<const __half*>(layer->o.weight),
                                          layer->vdim, static_cast<float*>(partial), T,
                                          layer->hidden, layer->vdim, 1, s);
    return et::run_linear(layer->o, b.z, static_cast<__half*>(partial), T, ET_ACT_NONE, b, s);
}

int et_encoder_after_attention_fwd(const et_encoder_layer_t* layer, const void* attn_sum,
                                   int sum_is_f32, const et_half* x, et_half* out, int batch,
                                   int seq, void* workspace, size_t workspace_bytes,
                                   et_stream stream) {
    int st = et::check_layer(layer);
    if (st != ET_OK) return st;
    if (!x || !out || !attn_sum || batch <= 0 || seq <= 0) return ET_ERR_INVALID_ARG;
    if (!workspace) return ET_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return ET_ERR_ALIGNMENT;
    const et::LayerBuffers b = et::carve(layer, batch, seq, workspace);
    if (workspace_bytes < b.total) return ET_ERR_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int T = batch * seq;
    const __half* xin = reinterpret_cast<const __half*>(x);
    const __half* g1 = reinterpret_cast<const __half*>(layer->ln1_gamma);
    const __half* b1 = reinterpret_cast<const __half*>(layer->ln1_beta);
    if (sum_is_f32) {
        if (layer->hidden > 2048) return ET_ERR_SHAPE;
        st = et::launch_skip_layernorm_partials(static_cast<const float*>(attn_sum), 1,
                                                static_cast<size_t>(T) * layer->hidden,
                                                reinterpret_cast<const __half*>(layer->o.bias), xin,
                                                g1, b1, b.y, T, layer->hidden, s);
    } else {
        st = et::launch_skip_layernorm(static_cast<const __half*>(attn_sum), xin, g1, b1, b.y, T,
                                       layer->hidden, s);
    }
    if (st != ET_OK) return st;
    return et::ffn_block(layer, b, T, reinterpret_cast<__half*>(out), s);
}

int et_encoder_ffn_fwd(const et_encoder_layer_t* layer, const et_half* y, et_half* out, int batch, int seq,
                       void* workspace, size_t workspace_bytes, et_stream stream) {
    int st = et::check_layer(layer);
    if (st != ET_OK) return st;
    if (!y || !out || batch <= 0 || seq <= 0) return ET_ERR_INVALID_ARG;
    if (!workspace) return ET_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return ET_ERR_ALIGNMENT;
    if (!et::aligned16(y)) return ET_ERR_ALIGNMENT;
    et::LayerBuffers b = et::carve(layer, batch, seq, workspace);
    if (workspace_bytes < b.total) return ET_ERR_WORKSPACE;
    b.y = const_cast<__half*>(reinterpret_cast<const __half*>(y));  // read only
    return et::ffn_block(layer, b, batch * seq, reinterpret_cast<__half*>(out),
                         static_cast<cudaStream_t>(stream));
}

}  // extern "C"
