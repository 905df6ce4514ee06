"""Pins the oracle and the host-side format builders to the committed golden fixtures
(tests/golden/, produced by make_golden.py from the reference's own Python helpers and from a
float64 PyTorch evaluation).  Index arrays must match bit-exactly."""
import os
import struct

import numpy as np

from conftest import errors

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _tile_cases(et):
    for i, (out, inn, sp) in enumerate([(64, 96, 0.5), (128, 64, 0.8), (48, 48, 0.0)]):
        w = et.synth.prune_tiles(et.synth.normal(31, i, (out, inn), 1.0), 31, 100 + i, sp)
        yield f"case{i}", w


def test_tile_csr_layout_matches_reference_exporter(et, orc):
    g = np.load(os.path.join(GOLD, "tile_csr_golden.npz"))
    for name, w in _tile_cases(et):
        for builder in (et.synth.dense_to_tile, orc.dense_to_tile):
            rp, ro, tiles = builder(w)
            assert rp.dtype == np.int32 and ro.dtype == np.int32
            assert np.array_equal(rp, g[name + "_row_ptr"]), name
            assert np.array_equal(ro, g[name + "_column"]), name
            assert np.array_equal(np.asarray(tiles, np.float32), g[name + "_data"]), name


def test_all_zero_matrix_gives_empty_tile_csr(et, orc):
    w = np.zeros((32, 160), np.float16)
    for builder in (et.synth.dense_to_tile, orc.dense_to_tile):
        rp, ro, tiles = builder(w)
        assert np.all(rp == 0) and len(ro) == 0 and len(tiles) == 0


def test_csr_file_layout(et, orc):
    blob = open(os.path.join(GOLD, "dense_4_3_csr.bin"), "rb").read()
    nrow, ncol, nnz = struct.unpack_from("III", blob, 0)
    assert (nrow, ncol, nnz) == (4, 3, 12) and len(blob) == 128
    indptr = np.frombuffer(blob, np.int32, nrow + 1, 12)
    indices = np.frombuffer(blob, np.int32, nnz, 12 + 4 * (nrow + 1))
    data = np.frombuffer(blob, np.float32, nnz, 12 + 4 * (nrow + 1) + 4 * nnz)
    ip, ix, dv = et.synth.dense_to_csr(np.ones((4, 3), np.float32))
    assert np.array_equal(ip, indptr) and np.array_equal(ix, indices) and np.array_equal(dv, data)
    ip2, ix2, dv2 = orc.dense_to_csr(np.ones((4, 3), np.float32))
    assert np.array_equal(ip2, indptr) and np.array_equal(ix2, indices) and np.array_equal(dv2, data)
    import ctypes
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    assert et.lib().et_validate_csr(vp(ip), vp(ix), 12, 3, 4) == 0


def test_row_file_layout(et):
    """uint32 nrow, ncol, len; uint32 ids[len]; float32 rows[len * ncol]."""
    blob = open(os.path.join(GOLD, "row_file_golden.bin"), "rb").read()
    nrow, ncol, n = struct.unpack_from("III", blob, 0)
    ids = np.frombuffer(blob, np.uint32, n, 12).astype(np.int32)
    rows = np.frombuffer(blob, np.float32, n * ncol, 12 + 4 * n).reshape(n, ncol)
    mat = et.synth.normal(41, 1, (nrow, ncol), 1.0).astype(np.float64)
    mat[et.synth.choose_ids(41, 2, nrow, 0.5, multiple=1)] = 0
    keep = np.nonzero(np.any(mat != 0, axis=1))[0].astype(np.int32)
    rid, r = et.synth.dense_to_row(mat.astype(np.float32), keep)
    assert (nrow, ncol) == (32, 16)
    assert np.array_equal(rid, ids) and np.array_equal(r, rows)


def test_oracle_encoder_matches_float64_pytorch(et, orc):
    g = np.load(os.path.join(GOLD, "encoder_torch_f64.npz"))
    cases = {"c1": (1, 128, 512, 8, 2048, 0), "small_causal": (2, 24, 64, 4, 128, 1),
             "small_padding": (3, 20, 64, 2, 96, 2)}
    for tag, (batch, seq, hidden, nhead, ff, mask_kind) in cases.items():
        w = et.synth.encoder_layer_weights(2021, 0, hidden, ff, bias_std=0.02 if tag != "c1" else 0.0,
                                           ln_noise=0.1 if tag != "c1" else 0.0)
        x = et.synth.normal(2021, 99, (batch * seq, hidden), 1.0)
        vl = np.array([seq, 7, 1], np.int32)[:batch] if mask_kind == 2 else None
        out = orc.encoder_layer(x, w, batch, seq, nhead, 2, mask_kind, None, vl)
        rel, mx = errors(out, g[tag])
        assert rel < 2e-6 and mx < 2e-5, (tag, rel, mx)
