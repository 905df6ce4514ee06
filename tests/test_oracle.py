"""Pins the CPU oracle (oracle/et_oracle.cpp): closed forms implied by the reference's
constant generators, independent float64 numpy evaluations of every operator, format-native
sparse loops against the densified dense evaluation."""
import numpy as np
import pytest

from conftest import errors


def _rand(et, seed, tid, shape, std=1.0):
    return et.synth.normal(seed, tid, shape, std).astype(np.float32)


def _gelu(x):
    return x * (0.5 + 0.5 * np.tanh(x * (0.035677408136300125 * x * x + 0.7978845608028654)))


def test_dense_closed_form(orc):
    # W = 1, x = 1, b = 0.5 -> in + 0.5 (Linear/gen_linear.hpp:15-23, test_cublas.cu:12-21)
    y = orc.linear_dense(np.ones((5, 48), np.float32), np.ones((32, 48), np.float32),
                         np.full(32, 0.5, np.float32))
    assert np.all(y == 48.5)


def test_dense_vs_numpy(et, orc):
    x, w, b = _rand(et, 1, 1, (37, 80)), _rand(et, 1, 2, (48, 80), 0.1), _rand(et, 1, 3, (48,))
    ref = x.astype(np.float64) @ w.astype(np.float64).T + b
    for act, f in ((0, lambda v: v), (1, lambda v: np.maximum(v, 0)), (2, _gelu)):
        rel, mx = errors(orc.linear_dense(x, w, b, act), f(ref))
        assert rel < 1e-6 and mx < 1e-5


def test_sparse_formats_match_dense(et, orc):
    T, inn, out = 19, 96, 64
    x, w, b = _rand(et, 2, 1, (T, inn)), _rand(et, 2, 2, (out, inn), 0.1), _rand(et, 2, 3, (out,))
    wt = et.synth.prune_tiles(w, 2, 4, 0.6)
    rp, ro, tiles = orc.dense_to_tile(wt)
    assert errors(orc.linear_tile(x, rp, ro, tiles, out, b, 2), orc.linear_dense(x, wt, b, 2))[1] < 1e-5
    assert np.array_equal(orc.tile_to_dense(rp, ro, tiles, out, inn), wt)
    wv = et.synth.prune_1x16(w, 2, 5, 0.7)
    ti, ri, data = orc.dense_to_1x16(wv)
    assert errors(orc.linear_1x16(x, ti, ri, data, out, b, 1), orc.linear_dense(x, wv, b, 1))[1] < 1e-5
    wc = w * et.synth.keep_exact(2, 6, out * inn, 0.8).reshape(out, inn)
    ip, ix, dv = orc.dense_to_csr(wc)
    assert errors(orc.linear_csr(x, ip, ix, dv, out, b, 0), orc.linear_dense(x, wc, b, 0))[1] < 1e-5
    rid = et.synth.choose_ids(2, 7, out, 0.5)
    wr = np.zeros_like(w)
    wr[rid] = w[rid]
    assert errors(orc.linear_row(x, rid, w[rid], out, b, 2), orc.linear_dense(x, wr, b, 2))[1] < 1e-5
    assert errors(orc.linear_row_compressed(x, rid, w[rid], b),
                  orc.linear_dense(x, wr, b, 0)[:, rid])[1] < 1e-5
    cid = et.synth.choose_ids(2, 8, inn, 0.5)
    wcol = np.zeros_like(w)
    wcol[:, cid] = w[:, cid]
    assert errors(orc.linear_col(x, cid, w[:, cid], b, 0), orc.linear_dense(x, wcol, b, 0))[1] < 1e-5


def test_layernorm(et, orc):
    x, s = _rand(et, 3, 1, (11, 72), 2.0), _rand(et, 3, 2, (11, 72))
    g, b = _rand(et, 3, 3, (72,)) + 1, _rand(et, 3, 4, (72,))
    v = (x + s).astype(np.float64)
    ref = (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-5) * g + b
    assert errors(orc.skip_layernorm(x, s, g, b), ref)[1] < 1e-5
    # constant row with gamma = beta = 0.2 -> 0.2 (SkipLayerNorm.cu:84-89 generator values)
    c = orc.skip_layernorm(np.full((2, 64), 0.2, np.float32), None, np.full(64, 0.2, np.float32),
                           np.full(64, 0.2, np.float32))
    assert np.allclose(c, 0.2, atol=1e-6)


def _attention_np(q, k, v, batch, seq, nhead, dq, dv, mask):
    out = np.zeros((batch * seq, nhead * dv))
    for b in range(batch):
        for h in range(nhead):
            Q = q[b * seq:(b + 1) * seq, h * dq:(h + 1) * dq].astype(np.float64)
            K = k[b * seq:(b + 1) * seq, h * dq:(h + 1) * dq].astype(np.float64)
            V = v[b * seq:(b + 1) * seq, h * dv:(h + 1) * dv].astype(np.float64)
            S = Q @ K.T / np.sqrt(dq) + mask[b]
            mx = S.max(1, keepdims=True)
            mx[~np.isfinite(mx)] = 0
            P = np.exp(S - mx)
            l = P.sum(1, keepdims=True)
            P = np.divide(P, l, out=np.zeros_like(P), where=l > 0)
            out[b * seq:(b + 1) * seq, h * dv:(h + 1) * dv] = P @ V
    return out


@pytest.mark.parametrize("mask_kind", [0, 1, 2, 3])
def test_attention_vs_numpy(et, orc, mask_kind):
    batch, seq, nhead, dq, dv = 2, 24, 3, 16, 32
    q, k = _rand(et, 4, 1, (batch * seq, nhead * dq)), _rand(et, 4, 2, (batch * seq, nhead * dq))
    v = _rand(et, 4, 3, (batch * seq, nhead * dv))
    vl = np.array([24, 5], np.int32)
    add = _rand(et, 4, 4, (seq, seq))
    add[2, :] = -np.inf
    mask = np.zeros((batch, seq, seq))
    if mask_kind == 1:
        mask[:] = np.where(np.tril(np.ones((seq, seq), bool)), 0, -np.inf)
    if mask_kind == 2:
        for b in range(batch):
            mask[b, :, vl[b]:] = -np.inf
    if mask_kind == 3:
        mask[:] = add
    z = orc.attention(q, k, v, batch, seq, nhead, dq, dv, mask_kind, add if mask_kind == 3 else None,
                      vl if mask_kind == 2 else None)
    assert errors(z, _attention_np(q, k, v, batch, seq, nhead, dq, dv, mask))[1] < 1e-5


def test_uniform_attention_closed_form(orc):
    # constant Q, K, V: Z = V (reference drivers feed constants; uniform softmax)
    seq, nhead, d = 16, 2, 16
    q = np.full((seq, nhead * d), 0.2, np.float32)
    assert np.allclose(orc.attention(q, q, q, 1, seq, nhead, d, d), 0.2, atol=1e-6)


def test_pruned_v_and_fused_vo(et, orc):
    batch, seq, nhead, dq, dv = 2, 20, 4, 16, 16
    T, vdim = batch * seq, nhead * dv
    q, k = _rand(et, 5, 1, (T, nhead * dq)), _rand(et, 5, 2, (T, nhead * dq))
    v = _rand(et, 5, 3, (T, vdim))
    col_id = et.synth.choose_ids(5, 4, vdim, 0.5, multiple=1)
    hp = et.synth.head_ptr_for(col_id, nhead, vdim)
    vz = np.zeros_like(v)
    vz[:, col_id] = v[:, col_id]
    z = orc.attention_pruned_v(q, k, v[:, col_id], col_id, hp, batch, seq, nhead, dq, dv, 1)
    assert errors(z, orc.attention(q, k, vz, batch, seq, nhead, dq, dv, 1))[1] < 1e-6
    # fused VO: sum_h P_h (X W_vo,h) + b_o  ==  O(attention(V)) when W_vo,h = W_v,h W_o,h
    em = 48
    x = _rand(et, 5, 5, (T, em))
    wv, wo = _rand(et, 5, 6, (vdim, em), 0.2), _rand(et, 5, 7, (em, vdim), 0.2)
    bo = _rand(et, 5, 8, (em,))
    vproj = x @ wv.T
    ref = orc.linear_dense(orc.attention(q, k, vproj, batch, seq, nhead, dq, dv), wo, bo)
    vo = np.zeros((batch, nhead, seq, em), np.float32)
    for h in range(nhead):
        w_vo = wv[h * dv:(h + 1) * dv].T @ wo[:, h * dv:(h + 1) * dv].T  # [em_in, em_out]
        vo[:, h] = (x @ w_vo).reshape(batch, seq, em)
    out = orc.fused_vo_attention(q, k, vo.reshape(-1, em), bo, batch, seq, nhead, dq, em)
    assert errors(out, ref)[0] < 1e-5


def test_encoder_layer_vs_composition(et, orc):
    batch, seq, hidden, nhead, ff = 2, 16, 64, 4, 128
    w = et.synth.encoder_layer_weights(6, 0, hidden, ff, std=0.1, bias_std=0.05, ln_noise=0.1)
    x = _rand(et, 6, 9, (batch * seq, hidden))
    wf = {k: v.astype(np.float32) for k, v in w.items()}
    qkv = orc.linear_dense(x, wf["wqkv"], wf["bqkv"])
    z = orc.attention(qkv[:, :hidden], qkv[:, hidden:2 * hidden], qkv[:, 2 * hidden:], batch, seq,
                      nhead, hidden // nhead, hidden // nhead, 1)
    y = orc.skip_layernorm(orc.linear_dense(z, wf["wo"], wf["bo"]), x, wf["ln1_g"], wf["ln1_b"])
    f = orc.linear_dense(y, wf["w1"], wf["b1"], 2)
    ref = orc.skip_layernorm(orc.linear_dense(f, wf["w2"], wf["b2"]), y, wf["ln2_g"], wf["ln2_b"])
    out = orc.encoder_layer(x, w, batch, seq, nhead, 2, 1)
    assert errors(out, ref)[1] < 1e-5
    out16 = orc.encoder_layer(x, w, batch, seq, nhead, 2, 1, round_mode=1)
    rel, mx = errors(out16, ref)
    assert 0 < rel < 5e-3 and mx < 2e-2
