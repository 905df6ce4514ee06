"""Weight import / export and preparation utilities (host code, CPU): the reference's on-disk
formats round-trip, the golden files written by the reference's own helpers parse, the fused
V.O weight reproduces attention + output projection, magnitude selection keeps what it should."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")


def test_layer_npz_round_trip_in_exporter_layout(et, tmp_path):
    hidden, ff = 64, 128
    w = et.synth.encoder_layer_weights(3, 0, hidden, ff, std=0.1, bias_std=0.05, ln_noise=0.1)
    for i, name in enumerate(("wqkv", "wo", "w1", "w2")):
        w[name] = et.synth.prune_tiles(w[name], 3, 10 + i, 0.5)
    names = et.weights.save_layer(str(tmp_path), 0, w)
    assert "transformer_encoder.layers.0.self_attn.in_proj_.npz" in names
    assert "transformer_encoder.layers.0.linear2..npz" in names
    assert open(tmp_path / "weights.txt").read().splitlines() == names
    z = np.load(tmp_path / names[0])
    assert sorted(z.files) == ["B", "column", "data", "row_ptr"]
    assert z["row_ptr"].dtype == np.int32 and z["column"].dtype == np.int32
    assert z["data"].dtype == np.float32 and z["data"].shape[1] == 256
    back = et.weights.load_layer(str(tmp_path), 0, {"wqkv": hidden, "wo": hidden, "w1": hidden, "w2": ff})
    for k, v in w.items():
        assert np.array_equal(back[k], v), k


def test_tile_npz_matches_reference_exporter_arrays(et, tmp_path):
    """save_tile_npz writes exactly the arrays the reference's gen_csr produced for the same
    matrices (golden file)."""
    g = np.load(os.path.join(GOLD, "tile_csr_golden.npz"))
    cases = [(64, 96, 0.5), (128, 64, 0.8), (48, 48, 0.0)]
    for i, (out, inn, sp) in enumerate(cases):
        w = et.synth.prune_tiles(et.synth.normal(31, i, (out, inn), 1.0), 31, 100 + i, sp)
        p = str(tmp_path / f"c{i}.npz")
        et.weights.save_tile_npz(p, w, np.zeros(out, np.float32))
        z = np.load(p)
        assert np.array_equal(z["row_ptr"], g[f"case{i}_row_ptr"])
        assert np.array_equal(z["column"], g[f"case{i}_column"])
        assert np.array_equal(z["data"], g[f"case{i}_data"])


def test_corrupt_npz_is_rejected(et, tmp_path):
    p = str(tmp_path / "bad.npz")
    np.savez(p, row_ptr=np.array([0, 2, 1], np.int32), column=np.array([0], np.int32),
             data=np.zeros((1, 256), np.float32), B=np.zeros(32, np.float32))
    with pytest.raises(ValueError):
        et.weights.load_tile_npz(p)


def test_raw_files_round_trip_and_golden(et, tmp_path):
    nrow, ids, rows = et.weights.read_row_file(os.path.join(GOLD, "row_file_golden.bin"))
    assert (nrow, rows.shape) == (32, (len(ids), 16)) and np.all(np.diff(ids) > 0)
    p = str(tmp_path / "x.row")
    et.weights.write_row_file(p, nrow, ids, rows)
    assert open(p, "rb").read() == open(os.path.join(GOLD, "row_file_golden.bin"), "rb").read()

    nr, nc, ip, ix, dv = et.weights.read_csr_file(os.path.join(GOLD, "dense_4_3_csr.bin"))
    assert (nr, nc, len(dv)) == (4, 3, 12) and np.array_equal(ip, [0, 3, 6, 9, 12])
    p = str(tmp_path / "x.csr")
    et.weights.write_csr_file(p, np.ones((4, 3), np.float32))
    assert open(p, "rb").read() == open(os.path.join(GOLD, "dense_4_3_csr.bin"), "rb").read()

    w = et.synth.normal(8, 1, (48, 64), 1.0).astype(np.float32)
    cid = et.synth.choose_ids(8, 2, 64, 0.5)
    _, cols = et.synth.dense_to_col(w, cid)
    p = str(tmp_path / "x.col")
    et.weights.write_col_file(p, 64, cid, cols)
    ncol, ids2, cols2 = et.weights.read_col_file(p)
    assert ncol == 64 and np.array_equal(ids2, cid) and np.array_equal(cols2, cols)
    with open(p, "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(ValueError):
        et.weights.read_col_file(p)


def test_w_vo_reproduces_attention_plus_output_projection(et, orc):
    batch, seq, nhead, dh, em = 2, 48, 4, 16, 64
    T = batch * seq
    x = et.synth.normal(12, 1, (T, em), 1.0)
    wq, wk, wv = (et.synth.normal(12, 2 + i, (nhead * dh, em), 0.2) for i in range(3))
    bv = et.synth.normal(12, 6, (nhead * dh,), 0.1)
    wo = et.synth.normal(12, 7, (em, nhead * dh), 0.2)
    bo = et.synth.normal(12, 8, (em,), 0.1)
    q = orc.linear_dense(x, wq, None, 0)
    k = orc.linear_dense(x, wk, None, 0)
    v = orc.linear_dense(x, wv, bv, 0)
    z = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 1)
    want = orc.linear_dense(z, wo, bo, 0)
    w_vo, b_vo = et.weights.build_w_vo(wv, bv, wo, nhead)
    assert w_vo.shape == (nhead, em, em) and b_vo.shape == (nhead, em)
    xf = x.astype(np.float32).reshape(batch, seq, em)
    vo = np.einsum("bse,heo->bhso", xf, w_vo.astype(np.float32)) + \
        b_vo.astype(np.float32)[None, :, None, :]
    got = orc.fused_vo_attention(q, k, vo.reshape(-1, em), bo, batch, seq, nhead, dh, em, 1)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel < 3e-3, rel   # W_VO is rounded to fp16 once


def test_magnitude_selection(et):
    w = et.synth.normal(21, 1, (96, 128), 1.0).astype(np.float32)
    w[16:32, 32:48] *= 100      # a tile that must survive
    w[0:16, 0:16] *= 1e-3       # a tile that must go
    p = et.weights.magnitude_prune_tiles(w, 0.75)
    t = p.reshape(6, 16, 8, 16)
    alive = (t != 0).any(axis=(1, 3))
    assert alive.sum() == 12 and alive[1, 2] and not alive[0, 0]
    norms = (w.reshape(6, 16, 8, 16) ** 2).sum(axis=(1, 3))
    assert norms[alive].min() >= norms[~alive].max()
    assert np.array_equal(p[alive.repeat(16, 0).repeat(16, 1)], w[alive.repeat(16, 0).repeat(16, 1)])

    v = et.weights.magnitude_prune_1x16(w, 0.9)
    assert ((v.reshape(96, 8, 16) != 0).any(axis=2)).sum() == round(0.1 * 96 * 8)

    rid = et.weights.magnitude_select_rows(w, 0.5)
    assert len(rid) == 48 and np.all(np.diff(rid) > 0)
    rn = (w ** 2).sum(axis=1)
    assert rn[rid].min() >= np.delete(rn, rid).max()
    cid = et.weights.magnitude_select_cols(w, 0.4)
    assert len(cid) == 64 and np.all(np.diff(cid) > 0)   # floor(128 * 0.6) = 76 -> 64
