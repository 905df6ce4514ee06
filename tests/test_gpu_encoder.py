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


def test_stack_of_three_layers_with_padding(et, orc, cuda):
    batch, seq, hidden, nhead, ff = 3, 96, 256, 4, 512
    ws = [et.synth.encoder_layer_weights(7, l, hidden, ff, std=0.05, bias_std=0.02, ln_noise=0.1)
          for l in range(3)]
    x = et.synth.normal(7, 97, (batch * seq, hidden), 1.0)
    vl = np.array([96, 40, 7], dtype=np.int32)
    y = _run(et, cuda, ws, x, batch, seq, nhead, mask_kind=2, valid_len=vl)
    ref = _oracle_stack(orc, ws, x, batch, seq, nhead, 2, vl)
    assert_close(y, ref, "3-layer stack with padding mask", rel_tol=8e-3, abs_tol=4e-2)


def test_pruned_qk_head_width(et, orc, cuda):
    """Attention-aware pruning: 16 of the 64 Q/K features of every head removed (dh_qk 48)."""
    batch, seq, hidden, nhead, ff = 2, 128, 768, 12, 1024
    w = et.synth.encoder_layer_weights(11, 0, hidden, ff, kdim=12 * 48, vdim=768)
    x = et.synth.normal(11, 96, (batch * seq, hidden), 1.0)
    assert_close(_run(et, cuda, [w], x, batch, seq, nhead),
                 _oracle_stack(orc, [w], x, batch, seq, nhead), "dh_qk 48")
