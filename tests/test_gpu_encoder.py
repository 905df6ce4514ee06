"""GPU parity of the whole encoder layer / stack through et_encoder_layer_fwd."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _run(et, cuda, ws, x, batch, seq, nhead, tile_sparse=False, mask_kind=0, valid_len=None):
    import torch
    layers = [et.EncoderLayer(w, nhead, et.ACT_GELU, device=cuda, tile_sparse=tile_sparse)
              for w in ws]
    stack = et.EncoderStack(layers, batch, seq, device=cuda)
    vl = None if valid_len is None else torch.from_numpy(valid_len).to(cuda)
    y = stack.forward(torch.from_numpy(x).to(cuda), mask_kind, None, vl)
    assert et.device_error() == 0
    return y.float().cpu().numpy()


def _oracle_stack(orc, ws, x, batch, seq, nhead, mask_kind=0, valid_len=None):
    cur = x.astype(np.float32)
    for w in ws:
        cur = orc.encoder_layer(cur, w, batch, seq, nhead, 2, mask_kind, None, valid_len)
    return cur


def test_layer_config1_shapes(et, orc, cuda):
    """d_model 512, 8 heads, FFN 2048, seq 128, batch 1 (the CPU-runnable configuration)."""
    batch, seq, hidden, nhead, ff = 1, 128, 512, 8, 2048
    w = et.synth.encoder_layer_weights(2021, 0, hidden, ff)
    x = et.synth.normal(2021, 99, (batch * seq, hidden), 1.0)
    y = _run(et, cuda, [w], x, batch, seq, nhead)
    assert_close(y, _oracle_stack(orc, [w], x, batch, seq, nhead), "config 1 layer",
                 dump="enc_c1")


def test_bert_base_layer_dense_and_tile(et, orc, cuda):
    batch, seq, hidden, nhead, ff = 4, 128, 768, 12, 3072
    w = et.synth.encoder_layer_weights(2021, 1, hidden, ff, bias_std=0.02, ln_noise=0.05)
    x = et.synth.normal(2021, 98, (batch * seq, hidden), 1.0)
    ref = _oracle_stack(orc, [w], x, batch, seq, nhead)
    assert_close(_run(et, cuda, [w], x, batch, seq, nhead), ref, "bert-base dense", dump="enc_bb")
    wp = dict(w)
    for i, name in enumerate(("wqkv", "wo", "w1", "w2")):
        wp[name] = et.synth.prune_tiles(w[name], 2021, 50 + i, 0.8)
    refp = _oracle_stack(orc, [wp], x, batch, seq, nhead)
    assert_close(_run(et, cuda, [wp], x, batch, seq, nhead, tile_sparse=True), refp,
                 "bert-base tile 80%", dump="enc_bb_tile")
    assert_close(_run(et, cuda, [wp], x, batch, seq, nhead, tile_sparse="unpacked"), refp,
                 "bert-base tile 80%, tile-CSR order")
    assert_close(_run(et, cuda, [wp], x, batch, seq, nhead, tile_sparse="auto"), refp,
                 "bert-base tile 80%, plan-time choice")


@pytest.mark.parametrize("splits", [1, 2, 3, -2])
def test_ffn2_split_k_forms(et, orc, cuda, splits):
    """FFN2 as split-K partial sums reduced inside the LayerNorm: single-CTA slices (2, 3) and
    CTA-pair slices (-2) against the unsplit layer (1) and the oracle."""
    import ctypes
    batch, seq, hidden, nhead, ff = 4, 128, 768, 12, 3072
    w = et.synth.encoder_layer_weights(2021, 2, hidden, ff, bias_std=0.02, ln_noise=0.05)
    x = et.synth.normal(2021, 94, (batch * seq, hidden), 1.0)
    try:
        et.lib().et_debug_set_ln_fusion(ctypes.c_int(0))  # the split forms feed the LayerNorm
        et.lib().et_debug_force_ffn2_splits(ctypes.c_int(splits))
        y = _run(et, cuda, [w], x, batch, seq, nhead)
    finally:
        et.lib().et_debug_force_ffn2_splits(ctypes.c_int(0))
        et.lib().et_debug_set_ln_fusion(ctypes.c_int(-1))
    assert_close(y, _oracle_stack(orc, [w], x, batch, seq, nhead), f"ffn2 splits {splits}")


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("batch,seq,hidden,nhead,ff", [(4, 128, 768, 12, 3072),
                                                       (3, 100, 1024, 16, 4096),
                                                       (2, 200, 256, 4, 512)])
def test_linear_layernorm_fusion_modes(et, orc, cuda, mode, batch, seq, hidden, nhead, ff):
    """O projection / FFN2 fused with their skip-LayerNorm (mask 1 / 2) against the separate
    kernels (0) and the oracle; a padding mask so that sequences differ."""
    import ctypes
    w = et.synth.encoder_layer_weights(2021, 3, hidden, ff, bias_std=0.02, ln_noise=0.05)
    x = et.synth.normal(2021, 93, (batch * seq, hidden), 1.0)
    vl = np.array([seq - 7 * i for i in range(batch)], dtype=np.int32)
    try:
        et.lib().et_debug_set_ln_fusion(ctypes.c_int(mode))
        y = _run(et, cuda, [w, w], x, batch, seq, nhead, mask_kind=2, valid_len=vl)
    finally:
        et.lib().et_debug_set_ln_fusion(ctypes.c_int(-1))
    assert_close(y, _oracle_stack(orc, [w, w], x, batch, seq, nhead, 2, vl),
                 f"linear+LN fusion mode {mode}")


def test_stack_of_three_layers_with_padding(et, orc, cuda):
    batch, seq, hidden, nhead, ff = 3, 96, 256, 4, 512
    ws = [et.synth.encoder_layer_weights(7, l, hidden, ff, std=0.05, bias_std=0.02, ln_noise=0.1)
          for l in range(3)]
    x = et.synth.normal(7, 97, (batch * seq, hidden), 1.0)
    vl = np.array([96, 40, 7], dtype=np.int32)
    y = _run(et, cuda, ws, x, batch, seq, nhead, mask_kind=2, valid_len=vl)
    ref = _oracle_stack(orc, ws, x, batch, seq, nhead, 2, vl)
    assert_close(y, ref, "3-layer stack with padding mask")


def test_pruned_qk_head_width(et, orc, cuda):
    """Attention-aware pruning: 16 of the 64 Q/K features of every head removed (dh_qk 48)."""
    batch, seq, hidden, nhead, ff = 2, 128, 768, 12, 1024
    w = et.synth.encoder_layer_weights(11, 0, hidden, ff, kdim=12 * 48, vdim=768)
    x = et.synth.normal(11, 96, (batch * seq, hidden), 1.0)
    assert_close(_run(et, cuda, [w], x, batch, seq, nhead),
                 _oracle_stack(orc, [w], x, batch, seq, nhead), "dh_qk 48")


def test_mixed_format_layer_bert_large_shapes(et, orc, cuda):
    """The BERT-large case of the paper's Table-2 style sweeps, composed from the per-operator
    entry points the C++ Encoder<config> template would bind: 1x16-pruned Q/K/V and O
    projections (90 %), row-pruned FFN-in and column-pruned FFN-out (50 %), padding mask,
    seq 384.  The oracle runs the format-native loops of the same operators."""
    import torch
    batch, seq, hidden, nhead, ff = 2, 384, 1024, 16, 4096
    T, dh = batch * seq, hidden // nhead
    w = et.synth.encoder_layer_weights(31, 0, hidden, ff, std=0.05, bias_std=0.02, ln_noise=0.1)
    x = et.synth.normal(31, 95, (T, hidden), 1.0)
    vl = np.array([384, 150], dtype=np.int32)
    wqkv = et.synth.prune_1x16(w["wqkv"], 31, 60, 0.9)
    wo = et.synth.prune_1x16(w["wo"], 31, 61, 0.9)
    rid = et.synth.choose_ids(31, 62, ff, 0.5)       # FFN-in keeps these output rows
    cid = rid                                        # FFN-out reads exactly those features
    q16, o16 = et.synth.dense_to_1x16(wqkv), et.synth.dense_to_1x16(wo)
    r_id, r_rows = et.synth.dense_to_row(w["w1"], rid)
    c_id, c_cols = et.synth.dense_to_col(w["w2"], cid)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)

    # ---- GPU ----
    xd = d(x)
    qkv = et.linear_1x16(xd, d(q16[0]), d(q16[1]), d(q16[2]), 3 * hidden, d(w["bqkv"]))
    z = et.attention(qkv[:, :hidden], qkv[:, hidden:2 * hidden], qkv[:, 2 * hidden:], batch, seq,
                     nhead, dh, dh, et.MASK_PADDING, None, d(vl))
    a = et.linear_1x16(z, d(o16[0]), d(o16[1]), d(o16[2]), hidden, d(w["bo"]))
    y = et.skip_layernorm(a, xd, d(w["ln1_g"]), d(w["ln1_b"]))
    f = et.linear_row_compressed(y, d(r_id), d(r_rows), d(w["b1"]))   # [T, nn_row], bias of kept rows
    f = et.act(f, et.ACT_GELU)
    a2 = et.linear_dense(f, d(c_cols), d(w["b2"]))                     # cols[out, nn_col] on the compressed input
    out = et.skip_layernorm(a2, y, d(w["ln2_g"]), d(w["ln2_b"]))
    assert et.device_error() == 0

    # ---- oracle, same operators (activations rounded to fp16 between operators as on the GPU) ----
    r16 = orc.round_fp16
    oq = r16(orc.linear_1x16(x, q16[0], q16[1], q16[2].astype(np.float32), 3 * hidden, w["bqkv"]))
    oz = r16(orc.attention(oq[:, :hidden], oq[:, hidden:2 * hidden], oq[:, 2 * hidden:], batch, seq,
                           nhead, dh, dh, 2, None, vl))
    oa = r16(orc.linear_1x16(oz, o16[0], o16[1], o16[2].astype(np.float32), hidden, w["bo"]))
    oy = r16(orc.skip_layernorm(oa, x, w["ln1_g"], w["ln1_b"]))
    of = r16(orc.act(r16(orc.linear_row_compressed(oy, r_id, r_rows.astype(np.float32), w["b1"])), 2))
    oa2 = r16(orc.linear_dense(of, c_cols.astype(np.float32), w["b2"]))
    ref = orc.skip_layernorm(oa2, oy, w["ln2_g"], w["ln2_b"])
    assert_close(out.float().cpu().numpy(), ref, "mixed-format BERT-large layer")

    # the same FFN through the scatter / gather forms of the row- and column-pruned Linear
    f_full = et.linear_row(y, d(r_id), d(r_rows), ff, d(w["b1"]), et.ACT_GELU)
    a3 = et.linear_col(f_full, d(c_id), d(c_cols), d(w["b2"]))
    assert et.device_error() == 0
    assert_close(a3.float().cpu().numpy(), a2.float().cpu().numpy(), "row scatter + col gather FFN",
                 rel_tol=2e-3, abs_tol=1e-2)


def test_host_pipeline_matches_resident_forward(et, cuda):
    """The serving loop (pinned host batches in and out, copies overlapped with compute over
    two slots) returns, for every batch of a stream of different batches, exactly what the
    resident forward returns."""
    import torch
    batch, seq, hidden, nhead, ff = 2, 64, 256, 4, 512
    ws = [et.synth.encoder_layer_weights(9, l, hidden, ff, std=0.05) for l in range(2)]
    layers = [et.EncoderLayer(w, nhead, et.ACT_GELU, device=cuda) for w in ws]
    stack = et.EncoderStack(layers, batch, seq, device=cuda)
    xs = [torch.from_numpy(et.synth.normal(9, 200 + i, (batch * seq, hidden), 1.0)).pin_memory()
          for i in range(5)]
    want = [stack.forward(x.to(cuda)).clone().cpu() for x in xs]
    pipe = et.HostPipeline(stack, depth=2)
    ys = [torch.empty_like(x).pin_memory() for x in xs]
    for x, y in zip(xs, ys):
        pipe.submit(x, y)
    pipe.drain()
    assert et.device_error() == 0
    for i, (y, w) in enumerate(zip(ys, want)):
        assert torch.equal(y, w), f"batch {i} differs"


def test_repeated_forwards_agree(et, orc, cuda):
    """Dependent launches start kernels before their predecessors finish; a buffer a predecessor
    writes must never be read through a non-coherent path.  Forty forwards of a short stack
    (few CTAs per kernel, so that several kernels are resident at once) must all agree."""
    import torch
    batch, seq, hidden, nhead, ff = 4, 128, 768, 12, 3072
    w = et.synth.encoder_layer_weights(2021, 3, hidden, ff, bias_std=0.02, ln_noise=0.05)
    x = et.synth.normal(2021, 93, (batch * seq, hidden), 1.0)
    layers = [et.EncoderLayer(w, nhead, et.ACT_GELU, device=cuda) for _ in range(2)]
    stack = et.EncoderStack(layers, batch, seq, device=cuda)
    xd = torch.from_numpy(x).to(cuda)
    outs = [stack.forward(xd).clone() for _ in range(40)]
    torch.cuda.synchronize()
    assert et.device_error() == 0
    assert all(torch.equal(o, outs[0]) for o in outs[1:])
    assert_close(outs[0].float().cpu().numpy(), _oracle_stack(orc, [w, w], x, batch, seq, nhead),
                 "two-layer stack, repeated")
