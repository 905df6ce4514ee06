// GPU test of the C++ host API that mirrors the reference's operator classes
// (scpaper-2021_b200/host/): the reference's own drivers build operators from constant
// generators and print one value (Linear/test/test_tile.cu:56-75, test/main.cu); here the
// same constructions are checked against closed forms and against the CPU oracle.
// Exit code 0 = all checks passed.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../scpaper-2021_b200/host/Encoder/Encoder.h"

// ---- CPU oracle (test infrastructure), linked from oracle/libet_oracle.so ----
extern "C" {
void orc_linear_dense(const float*, const float*, const float*, float*, int, int, int, int);
void orc_attention(const float*, const float*, const float*, float*, int, int, int, int, int, int,
                   int, int, int, int, const float*, const int*, float);
void orc_attention_pruned_v(const float*, const float*, const float*, const int*, const int*, int,
                            float*, int, int, int, int, int, int, int, int, int, const float*,
                            const int*, float);
void orc_fused_vo_attention(const float*, const float*, const float*, const float*, float*, int,
                            int, int, int, int, int, int, int, const float*, const int*, float);
void orc_encoder_layer(const float*, float*, int, int, int, int, int, int, int, const float*,
                       const float*, const float*, const float*, const float*, const float*,
                       const float*, const float*, const float*, const float*, const float*,
                       const float*, int, int, const float*, const int*, int);
int orc_dense_to_tile(const float*, int, int, int*, int*, float*);
int orc_dense_to_1x16(const float*, int, int, int*, int*, float*);
}

static int g_failures = 0;
#define CHECK(cond, ...)                 \
    do {                                 \
        if (!(cond)) {                   \
            ++g_failures;                \
            std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);    \
            std::printf("\n");           \
        }                                \
    } while (0)

static uint64_t g_rng = 12345;
static float nrand(float std) {
    // Box-Muller on SplitMix64 bits
    const double u1 = ((et_host::splitmix64(g_rng) >> 11) + 0.5) / 9007199254740992.0;
    const double u2 = ((et_host::splitmix64(g_rng) >> 11) + 0.5) / 9007199254740992.0;
    const float v = (float)(std * std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
    return __half2float(__float2half_rn(v));  // fp16-representable
}
static std::vector<float> nvec(size_t n, float std) {
    std::vector<float> v(n);
    for (auto& x : v) x = nrand(std);
    return v;
}
static std::vector<half> to_half(const std::vector<float>& v) {
    std::vector<half> h(v.size());
    for (size_t i = 0; i < v.size(); ++i) h[i] = __float2half_rn(v[i]);
    return h;
}
static std::vector<float> to_float(const culib::CUDA_ptr<half>& d) {
    std::vector<half> h = d.to_host();
    std::vector<float> f(h.size());
    for (size_t i = 0; i < h.size(); ++i) f[i] = __half2float(h[i]);
    return f;
}
static void compare(const std::vector<float>& got, const std::vector<float>& ref, const char* what,
                    double rel_tol = 5e-3, double abs_tol = 2e-2) {
    double num = 0, den = 0, mx = 0;
    for (size_t i = 0; i < ref.size(); ++i) {
        const double d = (double)got[i] - ref[i];
        num += d * d;
        den += (double)ref[i] * ref[i];
        mx = std::fmax(mx, std::fabs(d));
    }
    const double rel = std::sqrt(num / std::fmax(den, 1e-30));
    std::printf("%-44s rel-L2 %.3e  max-abs %.3e\n", what, rel, mx);
    CHECK(rel <= rel_tol && mx <= abs_tol && std::isfinite(rel), "%s out of tolerance", what);
}
static int device_error() {
    int code = -1;
    etChk(et_device_error(&code));
    return code;
}

// W = 1, x = 1, b = 0.5: every output equals (number of surviving weights of its row) + 0.5
template <typename MAT> static void closed_form_linear(const char* name, float sparsity) {
    const int in = 256, out = 128, size = 96;
    auto lin = gen_sparse_linear<MAT>(out, in, size, sparsity);
    culib::CUDA_ptr<half> x((size_t)size * in, __float2half_rn(1.0f)), y((size_t)size * out);
    lin->forward(y.get(), x.get());
    CHECK(device_error() == 0, "device error");
    auto f = to_float(y);
    // the dense count per output row, from a second forward with a one-hot probe is overkill:
    // compare row 0 and row size-1 (all token rows are identical) and integrality instead
    bool same = true, integral = true;
    double total = 0;
    for (int o = 0; o < out; ++o) {
        same = same && f[o] == f[(size_t)(size - 1) * out + o];
        const float w = f[o] - 0.5f;
        integral = integral && w == std::floor(w) && w >= 0 && w <= in;
        total += w;
    }
    CHECK(same && integral, "%s: rows differ or non-integral weight counts", name);
    if (sparsity == 0.f) CHECK(total == (double)in * out, "%s dense: expected in + 0.5 everywhere", name);
    std::printf("%-12s s=%.2f  surviving weights seen through y: %.0f of %d\n", name, sparsity, total,
                in * out);
}

static void test_norms() {
    const int size = 768, rows = 33;
    auto ln = gen_skLN(size);
    culib::CUDA_ptr<half> a((size_t)rows * size, __float2half_rn(0.2f)), o((size_t)rows * size);
    ln->forward(o.get(), a.get(), a.get(), rows);
    auto f = to_float(o);
    bool ok = true;
    for (float v : f) ok = ok && std::fabs(v - 0.2f) < 2e-3f;
    CHECK(ok, "skip-LN of a constant row must return beta");
    auto ln2 = gen_LN(size);
    ln2->forward(o.get(), a.get(), rows);
    CHECK(device_error() == 0, "device error");
}

struct LayerW {
    std::vector<float> wqkv, bqkv, wo, bo, w1, b1, w2, b2, g1, be1, g2, be2;
};
static void prune_tiles(std::vector<float>& w, int out, int in, float sparsity, uint64_t seed) {
    const int nbr = out / 16, nbc = in / 16;
    auto drop = et_host::sample_ids(nbr * nbc, (int)(nbr * nbc * sparsity), seed);
    for (int id : drop)
        for (int r = 0; r < 16; ++r)
            for (int c = 0; c < 16; ++c) w[(size_t)((id / nbc) * 16 + r) * in + (id % nbc) * 16 + c] = 0.f;
}
static tile_mat make_tile(const std::vector<float>& w, int out, int in) {
    const int n = orc_dense_to_tile(w.data(), out, in, nullptr, nullptr, nullptr);
    std::vector<int> rp(out / 16 + 1), ro(n);
    std::vector<float> tiles((size_t)n * 256);
    orc_dense_to_tile(w.data(), out, in, rp.data(), ro.data(), tiles.data());
    CHECK(et_validate_tile_mat(rp.data(), ro.data(), n, in, out) == ET_OK, "tile validator");
    return tile_mat(rp, ro, to_half(tiles), in / 16);
}

// Encoder<tile-pruned, fused-QKV single-kernel attention, GELU> against the oracle layer
static void test_encoder_tile(int batch, int seq, int mask_kind) {
    const int hidden = 256, nhead = 4, ff = 512, T = batch * seq;
    auto model = std::make_shared<Model_t>(Model_t{hidden, hidden, seq, nhead, ff, hidden, 1, batch, mask_kind});
    LayerW w;
    w.wqkv = nvec((size_t)3 * hidden * hidden, 0.05f);
    w.wo = nvec((size_t)hidden * hidden, 0.05f);
    w.w1 = nvec((size_t)ff * hidden, 0.05f);
    w.w2 = nvec((size_t)hidden * ff, 0.05f);
    prune_tiles(w.wqkv, 3 * hidden, hidden, 0.5f, 1);
    prune_tiles(w.wo, hidden, hidden, 0.5f, 2);
    prune_tiles(w.w1, ff, hidden, 0.8f, 3);
    prune_tiles(w.w2, hidden, ff, 0.8f, 4);
    w.bqkv = nvec(3 * hidden, 0.02f);
    w.bo = nvec(hidden, 0.02f);
    w.b1 = nvec(ff, 0.02f);
    w.b2 = nvec(hidden, 0.02f);
    w.g1 = nvec(hidden, 0.1f);
    w.g2 = nvec(hidden, 0.1f);
    for (auto& g : w.g1) g = __half2float(__float2half_rn(g + 1.f));
    for (auto& g : w.g2) g = __half2float(__float2half_rn(g + 1.f));
    w.be1 = nvec(hidden, 0.1f);
    w.be2 = nvec(hidden, 0.1f);
    auto x = nvec((size_t)T * hidden, 1.0f);

    using attn_cfg = Attention_config<tile_mat, tile_mat, tile_mat, tile_mat, OTF_attn_full, true, false>;
    using enc_cfg = Encoder_config<attn_cfg, tile_mat, tile_mat, GELU_OP>;
    auto hb = [&](const std::vector<float>& b) { return to_half(b); };
    auto lqkv = std::make_unique<Linear<tile_mat>>(hidden, 3 * hidden, make_tile(w.wqkv, 3 * hidden, hidden), hb(w.bqkv).data(), T);
    auto lo = std::make_unique<Linear<tile_mat>>(hidden, hidden, make_tile(w.wo, hidden, hidden), hb(w.bo).data(), T);
    auto l1 = std::make_unique<Linear<tile_mat>>(hidden, ff, make_tile(w.w1, ff, hidden), hb(w.b1).data(), T);
    auto l2 = std::make_unique<Linear<tile_mat>>(ff, hidden, make_tile(w.w2, hidden, ff), hb(w.b2).data(), T);
    auto attn = std::make_unique<Attention<attn_cfg>>(std::move(lqkv), std::move(lo), model);
    auto ln1 = std::make_unique<SkipLayerNorm>(hb(w.g1).data(), hb(w.be1).data(), hidden);
    auto ln2 = std::make_unique<SkipLayerNorm>(hb(w.g2).data(), hb(w.be2).data(), hidden);
    Encoder<enc_cfg> enc(std::move(attn), std::move(ln1), std::move(ln2), std::move(l1), std::move(l2), model);

    culib::CUDA_ptr<half> dx(to_half(x)), dout((size_t)T * hidden);
    enc.forward(dout.get(), dx.get());
    enc.forward(dout.get(), dx.get());  // operators are reusable
    CHECK(device_error() == 0, "device error");
    std::vector<float> ref((size_t)T * hidden);
    orc_encoder_layer(x.data(), ref.data(), batch, seq, hidden, nhead, hidden, hidden, ff, w.wqkv.data(),
                      w.bqkv.data(), w.wo.data(), w.bo.data(), w.w1.data(), w.b1.data(), w.w2.data(),
                      w.b2.data(), w.g1.data(), w.be1.data(), w.g2.data(), w.be2.data(), 2, mask_kind,
                      nullptr, nullptr, 0);
    char what[96];
    std::snprintf(what, sizeof what, "Encoder<tile, fused QKV> b%d s%d mask%d", batch, seq, mask_kind);
    compare(to_float(dout), ref, what);
}

// Encoder<dense weights, fused-QKV single-kernel attention, GELU>: the O projection and FFN2 run
// with their SkipLayerNorm in the GEMM epilogue (one kernel each) when the library expects that
// to pay, the separate kernels otherwise; both against the oracle layer.
static void test_encoder_dense(int batch, int seq, int mask_kind) {
    const int hidden = 256, nhead = 4, ff = 512, T = batch * seq;
    auto model = std::make_shared<Model_t>(Model_t{hidden, hidden, seq, nhead, ff, hidden, 1, batch, mask_kind});
    LayerW w;
    w.wqkv = nvec((size_t)3 * hidden * hidden, 0.05f);
    w.wo = nvec((size_t)hidden * hidden, 0.05f);
    w.w1 = nvec((size_t)ff * hidden, 0.05f);
    w.w2 = nvec((size_t)hidden * ff, 0.05f);
    w.bqkv = nvec(3 * hidden, 0.02f);
    w.bo = nvec(hidden, 0.02f);
    w.b1 = nvec(ff, 0.02f);
    w.b2 = nvec(hidden, 0.02f);
    w.g1 = nvec(hidden, 0.1f);
    w.g2 = nvec(hidden, 0.1f);
    for (auto& g : w.g1) g = __half2float(__float2half_rn(g + 1.f));
    for (auto& g : w.g2) g = __half2float(__float2half_rn(g + 1.f));
    w.be1 = nvec(hidden, 0.1f);
    w.be2 = nvec(hidden, 0.1f);
    auto x = nvec((size_t)T * hidden, 1.0f);

    using attn_cfg = Attention_config<base_mat, base_mat, base_mat, base_mat, OTF_attn_full, true, false>;
    using enc_cfg = Encoder_config<attn_cfg, base_mat, base_mat, GELU_OP>;
    auto hb = [&](const std::vector<float>& b) { return to_half(b); };
    auto dense = [&](const std::vector<float>& m) { return base_mat(to_half(m)); };
    auto lqkv = std::make_unique<Linear<base_mat>>(hidden, 3 * hidden, dense(w.wqkv), hb(w.bqkv).data(), T);
    auto lo = std::make_unique<Linear<base_mat>>(hidden, hidden, dense(w.wo), hb(w.bo).data(), T);
    auto l1 = std::make_unique<Linear<base_mat>>(hidden, ff, dense(w.w1), hb(w.b1).data(), T);
    auto l2 = std::make_unique<Linear<base_mat>>(ff, hidden, dense(w.w2), hb(w.b2).data(), T);
    auto attn = std::make_unique<Attention<attn_cfg>>(std::move(lqkv), std::move(lo), model);
    auto ln1 = std::make_unique<SkipLayerNorm>(hb(w.g1).data(), hb(w.be1).data(), hidden);
    auto ln2 = std::make_unique<SkipLayerNorm>(hb(w.g2).data(), hb(w.be2).data(), hidden);
    Encoder<enc_cfg> enc(std::move(attn), std::move(ln1), std::move(ln2), std::move(l1), std::move(l2), model);

    CHECK(et_linear_skip_layernorm_pays(T, ff, hidden) == 1, "fused Linear + LayerNorm expected to pay here");
    culib::CUDA_ptr<half> dx(to_half(x)), dout((size_t)T * hidden);
    enc.forward(dout.get(), dx.get());
    enc.forward(dout.get(), dx.get());
    CHECK(device_error() == 0, "device error");
    std::vector<float> ref((size_t)T * hidden);
    orc_encoder_layer(x.data(), ref.data(), batch, seq, hidden, nhead, hidden, hidden, ff, w.wqkv.data(),
                      w.bqkv.data(), w.wo.data(), w.bo.data(), w.w1.data(), w.b1.data(), w.w2.data(),
                      w.b2.data(), w.g1.data(), w.be1.data(), w.g2.data(), w.be2.data(), 2, mask_kind,
                      nullptr, nullptr, 0);
    char what[96];
    std::snprintf(what, sizeof what, "Encoder<dense, fused QKV, fused LN> b%d s%d mask%d", batch, seq, mask_kind);
    compare(to_float(dout), ref, what);
}

// Attention with three dense projections on side streams; Prune_attn with a row-pruned V
static void test_attention_variants() {
    const int batch = 2, seq = 128, hidden = 256, nhead = 4, T = batch * seq, dh = hidden / nhead;
    auto model = std::make_shared<Model_t>(Model_t{hidden, hidden, seq, nhead, 512, hidden, 1, batch, 1});
    auto wq = nvec((size_t)hidden * hidden, 0.05f), wk = nvec((size_t)hidden * hidden, 0.05f),
         wv = nvec((size_t)hidden * hidden, 0.05f), wo = nvec((size_t)hidden * hidden, 0.05f);
    auto bq = nvec(hidden, 0.02f), bk = nvec(hidden, 0.02f), bv = nvec(hidden, 0.02f), bo = nvec(hidden, 0.02f);
    auto x = nvec((size_t)T * hidden, 1.0f);
    std::vector<float> q((size_t)T * hidden), k(q.size()), v(q.size()), z(q.size()), ref(q.size());
    orc_linear_dense(x.data(), wq.data(), bq.data(), q.data(), T, hidden, hidden, 0);
    orc_linear_dense(x.data(), wk.data(), bk.data(), k.data(), T, hidden, hidden, 0);
    orc_linear_dense(x.data(), wv.data(), bv.data(), v.data(), T, hidden, hidden, 0);
    const float scale = 1.0f / std::sqrt((float)dh);
    orc_attention(q.data(), k.data(), v.data(), z.data(), batch, seq, nhead, dh, dh, hidden, hidden, hidden,
                  hidden, 1, nullptr, nullptr, scale);
    orc_linear_dense(z.data(), wo.data(), bo.data(), ref.data(), T, hidden, hidden, 0);
    culib::CUDA_ptr<half> dx(to_half(x)), dout((size_t)T * hidden);
    {
        using cfg = Attention_config<base_mat, base_mat, base_mat, base_mat, OTF_attn_full, false, true>;
        auto mk = [&](const std::vector<float>& w, const std::vector<float>& b) {
            return std::make_unique<Linear<base_mat>>(hidden, hidden, base_mat(to_half(w)), to_half(b).data(), T);
        };
        Attention<cfg> attn(mk(wq, bq), mk(wk, bk), mk(wv, bv), mk(wo, bo), model);
        attn.forward(dout.get(), dx.get(), dx.get(), dx.get());
        CHECK(device_error() == 0, "device error");
        compare(to_float(dout), ref, "Attention<dense x4, isPara> causal");
    }
    {
        // V projection row-pruned to half of its output features -> compressed V -> Prune_attn
        using cfg = Attention_config<base_mat, base_mat, row_mat, base_mat, Prune_attn, false, false>;
        auto ids = et_host::sample_ids(hidden, hidden / 2, 77);
        std::sort(ids.begin(), ids.end());
        std::vector<float> rows((size_t)ids.size() * hidden), vp(v.size(), 0.f), zp(z.size()), refp(ref.size());
        for (size_t i = 0; i < ids.size(); ++i)
            for (int c = 0; c < hidden; ++c) rows[i * hidden + c] = wv[(size_t)ids[i] * hidden + c];
        for (int t = 0; t < T; ++t)
            for (int id : ids) vp[(size_t)t * hidden + id] = v[(size_t)t * hidden + id];
        orc_attention(q.data(), k.data(), vp.data(), zp.data(), batch, seq, nhead, dh, dh, hidden, hidden,
                      hidden, hidden, 1, nullptr, nullptr, scale);
        orc_linear_dense(zp.data(), wo.data(), bo.data(), refp.data(), T, hidden, hidden, 0);
        auto mk = [&](const std::vector<float>& w, const std::vector<float>& b) {
            return std::make_unique<Linear<base_mat>>(hidden, hidden, base_mat(to_half(w)), to_half(b).data(), T);
        };
        auto lv = std::make_unique<Linear<row_mat>>(
            hidden, hidden, row_mat(culib::CUDA_ptr<int>(ids), culib::CUDA_ptr<half>(to_half(rows)), hidden, hidden),
            to_half(bv).data(), T);
        Attention<cfg> attn(mk(wq, bq), mk(wk, bk), std::move(lv), mk(wo, bo), model);
        attn.forward(dout.get(), dx.get(), dx.get(), dx.get());
        CHECK(device_error() == 0, "device error");
        compare(to_float(dout), refp, "Attention<Prune_attn, row-pruned V>");
    }
    {
        // pre-multiplied V.O: W_vo[h] = W_v,h^T W_o,h^T (fp32 on the host, then rounded)
        using cfg = Attention_config<base_mat, base_mat, base_mat, base_mat, OTF_fused_attn, false, false>;
        std::vector<float> wvo((size_t)nhead * hidden * hidden), bvo((size_t)nhead * hidden, 0.f);
        for (int h = 0; h < nhead; ++h)
            for (int i = 0; i < hidden; ++i)
                for (int o = 0; o < hidden; ++o) {
                    double s = 0;
                    for (int d = 0; d < dh; ++d)
                        s += (double)wv[(size_t)(h * dh + d) * hidden + i] * wo[(size_t)o * hidden + h * dh + d];
                    wvo[((size_t)h * hidden + i) * hidden + o] = __half2float(__float2half_rn((float)s));
                }
        std::vector<float> vo((size_t)batch * nhead * seq * hidden), refv(ref.size());
        for (int b = 0; b < batch; ++b)
            for (int h = 0; h < nhead; ++h) {
                std::vector<float> wt((size_t)hidden * hidden);  // [out, in] view of W_vo[h]
                for (int i = 0; i < hidden; ++i)
                    for (int o = 0; o < hidden; ++o) wt[(size_t)o * hidden + i] = wvo[((size_t)h * hidden + i) * hidden + o];
                orc_linear_dense(x.data() + (size_t)b * seq * hidden, wt.data(), nullptr,
                                 vo.data() + ((size_t)b * nhead + h) * seq * hidden, seq, hidden, hidden, 0);
            }
        orc_fused_vo_attention(q.data(), k.data(), vo.data(), bo.data(), refv.data(), batch, seq, nhead, dh,
                               hidden, hidden, hidden, 1, nullptr, nullptr, scale);
        auto mk = [&](const std::vector<float>& w, const std::vector<float>& b) {
            return std::make_unique<Linear<base_mat>>(hidden, hidden, base_mat(to_half(w)), to_half(b).data(), T);
        };
        auto lvo = std::make_unique<Linear_VO>(culib::CUDA_ptr<half>(to_half(wvo)), culib::CUDA_ptr<half>(to_half(bvo)), model);
        FusedAttention<cfg> fa(mk(wq, bq), mk(wk, bk), std::move(lvo), culib::CUDA_ptr<half>(to_half(bo)), model);
        fa.forward(dout.get(), dx.get(), dx.get(), dx.get());
        CHECK(device_error() == 0, "device error");
        compare(to_float(dout), refv, "FusedAttention<OTF_fused_attn>");
    }
}

// Attention<dense fused-QKV weight, single kernel>: projection and attention run as one launch
static void test_attention_fused_qkv_dense() {
    const int batch = 3, seq = 100, hidden = 256, nhead = 4, T = batch * seq, dh = hidden / nhead;
    auto model = std::make_shared<Model_t>(Model_t{hidden, hidden, seq, nhead, 512, hidden, 1, batch, 1});
    auto wqkv = nvec((size_t)3 * hidden * hidden, 0.05f), wo = nvec((size_t)hidden * hidden, 0.05f);
    auto bqkv = nvec(3 * hidden, 0.02f), bo = nvec(hidden, 0.02f);
    auto x = nvec((size_t)T * hidden, 1.0f);
    std::vector<float> qkv((size_t)T * 3 * hidden), z((size_t)T * hidden), ref(z.size());
    orc_linear_dense(x.data(), wqkv.data(), bqkv.data(), qkv.data(), T, hidden, 3 * hidden, 0);
    orc_attention(qkv.data(), qkv.data() + hidden, qkv.data() + 2 * hidden, z.data(), batch, seq, nhead, dh,
                  dh, 3 * hidden, 3 * hidden, 3 * hidden, hidden, 1, nullptr, nullptr,
                  1.0f / std::sqrt((float)dh));
    orc_linear_dense(z.data(), wo.data(), bo.data(), ref.data(), T, hidden, hidden, 0);
    using cfg = Attention_config<base_mat, base_mat, base_mat, base_mat, OTF_attn_full, true, false>;
    auto lqkv = std::make_unique<Linear<base_mat>>(hidden, 3 * hidden, base_mat(to_half(wqkv)),
                                                   to_half(bqkv).data(), T);
    auto lo = std::make_unique<Linear<base_mat>>(hidden, hidden, base_mat(to_half(wo)), to_half(bo).data(), T);
    Attention<cfg> attn(std::move(lqkv), std::move(lo), model);
    culib::CUDA_ptr<half> dx(to_half(x)), dout((size_t)T * hidden);
    attn.forward(dout.get(), dx.get(), dx.get(), dx.get());
    CHECK(device_error() == 0, "device error");
    compare(to_float(dout), ref, "Attention<dense fused QKV, single kernel>");
}

static void test_errors() {
    bool threw = false;
    try {
        culib::CUDA_ptr<half> x(16 * 24), y(16 * 16);
        base_mat w((size_t)16 * 24);
        std::vector<half> b(16);
        Linear<base_mat> lin(24, 16, std::move(w), b.data(), 16);  // in % 16 != 0
        lin.forward(y.get(), x.get());
    } catch (const std::runtime_error&) {
        threw = true;
    }
    CHECK(threw, "a bad shape must surface as an exception, not a launch");
    CHECK(device_error() == 0, "device error");
}


// The paper's BERT-large configuration through Encoder<config>: Q | K | V and O projections
// pruned to 1x16 vectors (90 %), FFN hidden units pruned by half (row-pruned first Linear,
// column-pruned second Linear over the same units), padding mask with per-sequence lengths,
// batch 8, seq 384.  The oracle evaluates the dense equivalents (pruned entries zero).
static void test_encoder_bert_large_mixed_formats() {
    const int batch = 8, seq = 384, hidden = 1024, nhead = 16, ff = 4096, T = batch * seq;
    auto model = std::make_shared<Model_t>(Model_t{hidden, hidden, seq, nhead, ff, hidden, 1, batch, ET_MASK_PADDING});
    LayerW w;
    auto prune_vectors = [](std::vector<float>& m, int out, int in, float sparsity, uint64_t seed) {
        const int nvec = out * (in / 16);
        for (int id : et_host::sample_ids(nvec, (int)(nvec * sparsity), seed)) {
            float* v = m.data() + (size_t)(id / (in / 16)) * in + (size_t)(id % (in / 16)) * 16;
            for (int c = 0; c < 16; ++c) v[c] = 0.f;
        }
    };
    auto make_1x16 = [](const std::vector<float>& m, int out, int in) {
        const int n = orc_dense_to_1x16(m.data(), out, in, nullptr, nullptr, nullptr);
        std::vector<int> tidx((size_t)(out / 16) * (in / 16 + 1)), ridx(n);
        std::vector<float> data((size_t)n * 16);
        orc_dense_to_1x16(m.data(), out, in, tidx.data(), ridx.data(), data.data());
        CHECK(et_validate_1x16(tidx.data(), ridx.data(), n, in, out) == ET_OK, "1x16 validator");
        return mat1x16(out, in, tidx, ridx, to_half(data));
    };
    w.wqkv = nvec((size_t)3 * hidden * hidden, 0.02f);
    w.wo = nvec((size_t)hidden * hidden, 0.02f);
    w.w1 = nvec((size_t)ff * hidden, 0.02f);
    w.w2 = nvec((size_t)hidden * ff, 0.02f);
    prune_vectors(w.wqkv, 3 * hidden, hidden, 0.9f, 11);
    prune_vectors(w.wo, hidden, hidden, 0.9f, 12);
    std::vector<int> kept = et_host::sample_ids(ff, ff / 2, 13);  // surviving hidden units of the FFN
    std::sort(kept.begin(), kept.end());
    std::vector<char> alive(ff, 0);
    for (int u : kept) alive[u] = 1;
    std::vector<float> rows((size_t)kept.size() * hidden), cols((size_t)hidden * kept.size());
    for (int u = 0; u < ff; ++u)
        if (!alive[u]) {
            for (int c = 0; c < hidden; ++c) w.w1[(size_t)u * hidden + c] = 0.f;
            for (int o = 0; o < hidden; ++o) w.w2[(size_t)o * ff + u] = 0.f;
        }
    for (size_t k = 0; k < kept.size(); ++k) {
        for (int c = 0; c < hidden; ++c) rows[k * hidden + c] = w.w1[(size_t)kept[k] * hidden + c];
        for (int o = 0; o < hidden; ++o) cols[(size_t)o * kept.size() + k] = w.w2[(size_t)o * ff + kept[k]];
    }
    w.bqkv = nvec(3 * hidden, 0.02f);
    w.bo = nvec(hidden, 0.02f);
    w.b1 = nvec(ff, 0.02f);
    w.b2 = nvec(hidden, 0.02f);
    w.g1 = nvec(hidden, 0.1f);
    w.g2 = nvec(hidden, 0.1f);
    for (auto& g : w.g1) g = __half2float(__float2half_rn(g + 1.f));
    for (auto& g : w.g2) g = __half2float(__float2half_rn(g + 1.f));
    w.be1 = nvec(hidden, 0.1f);
    w.be2 = nvec(hidden, 0.1f);
    auto x = nvec((size_t)T * hidden, 1.0f);
    std::vector<int> vl(batch);
    for (int b = 0; b < batch; ++b) vl[b] = 128 + (int)(et_host::splitmix64(g_rng) % 257);

    using attn_cfg = Attention_config<mat1x16, mat1x16, mat1x16, mat1x16, OTF_attn_full, true, false>;
    using enc_cfg = Encoder_config<attn_cfg, row_mat, col_mat, GELU_OP>;
    auto hb = [&](const std::vector<float>& b) { return to_half(b); };
    auto lqkv = std::make_unique<Linear<mat1x16>>(hidden, 3 * hidden, make_1x16(w.wqkv, 3 * hidden, hidden), hb(w.bqkv).data(), T);
    auto lo = std::make_unique<Linear<mat1x16>>(hidden, hidden, make_1x16(w.wo, hidden, hidden), hb(w.bo).data(), T);
    culib::CUDA_ptr<int> ids(kept);
    auto l1 = std::make_unique<Linear<row_mat>>(hidden, ff, row_mat(ids, culib::CUDA_ptr<half>(to_half(rows)), ff, hidden), hb(w.b1).data(), T);
    auto l2 = std::make_unique<Linear<col_mat>>(ff, hidden, col_mat(ids, culib::CUDA_ptr<half>(to_half(cols)), hidden, ff, (int)kept.size()), hb(w.b2).data(), T);
    auto attn = std::make_unique<Attention<attn_cfg>>(std::move(lqkv), std::move(lo), model);
    culib::CUDA_ptr<int> dvl(vl);
    attn->set_valid_len(dvl.get());
    auto ln1 = std::make_unique<SkipLayerNorm>(hb(w.g1).data(), hb(w.be1).data(), hidden);
    auto ln2 = std::make_unique<SkipLayerNorm>(hb(w.g2).data(), hb(w.be2).data(), hidden);
    Encoder<enc_cfg> enc(std::move(attn), std::move(ln1), std::move(ln2), std::move(l1), std::move(l2), model);
    culib::CUDA_ptr<half> dx(to_half(x)), dout((size_t)T * hidden);
    enc.forward(dout.get(), dx.get());
    CHECK(device_error() == 0, "device error");
    std::vector<float> ref((size_t)T * hidden);
    orc_encoder_layer(x.data(), ref.data(), batch, seq, hidden, nhead, hidden, hidden, ff, w.wqkv.data(),
                      w.bqkv.data(), w.wo.data(), w.bo.data(), w.w1.data(), w.b1.data(), w.w2.data(),
                      w.b2.data(), w.g1.data(), w.be1.data(), w.g2.data(), w.be2.data(), 2, ET_MASK_PADDING,
                      nullptr, vl.data(), 0);
    // padded query rows are computed but carry no meaning: compare the valid rows
    std::vector<float> got = to_float(dout), g2, r2;
    for (int b = 0; b < batch; ++b)
        for (int t = 0; t < vl[b]; ++t)
            for (int c = 0; c < hidden; ++c) {
                g2.push_back(got[((size_t)b * seq + t) * hidden + c]);
                r2.push_back(ref[((size_t)b * seq + t) * hidden + c]);
            }
    compare(g2, r2, "Encoder<1x16 | row | col> BERT-large b8 s384 padding");
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        std::printf("no CUDA device\n");
        return 2;
    }
    try {
        closed_form_linear<base_mat>("base_mat", 0.f);
        closed_form_linear<tile_mat>("tile_mat", 0.f);
        closed_form_linear<tile_mat>("tile_mat", 0.5f);   // expanded to dense at construction
        closed_form_linear<tile_mat>("tile_mat", 0.99f);  // sparse enough for the packed tile kernel
        closed_form_linear<row_mat>("row_mat", 0.5f);
        closed_form_linear<col_mat>("col_mat", 0.5f);
        closed_form_linear<mat1x16>("mat1x16", 0.9f);
        closed_form_linear<csr_mat>("csr_mat", 0.9f);
        test_norms();
        test_encoder_tile(2, 128, 1);
        test_encoder_tile(3, 80, 0);
        test_encoder_dense(2, 128, 1);
        test_encoder_dense(3, 100, 0);
        test_attention_variants();
        test_attention_fused_qkv_dense();
        test_encoder_bert_large_mixed_formats();
        test_errors();
    } catch (const std::exception& e) {
        std::printf("EXCEPTION: %s\n", e.what());
        return 3;
    }
    std::printf(g_failures ? "%d check(s) FAILED\n" : "all host-API checks passed\n", g_failures);
    return g_failures ? 1 : 0;
}
