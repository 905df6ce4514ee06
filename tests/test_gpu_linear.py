"""GPU parity of the Linear layers (all five weight formats + dense) through the C ABI
against the CPU oracle.  Shapes follow the reference's benchmarks: the four BERT-base GEMMs
768->2304, 768->768, 768->3072, 3072->768 (Linear/test/benchmark/test.sh:5-8) plus ragged and
tiny cases; sparsity sweep values from Linear/test/test_concurrent.cu:14-52."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _host(t):
    return t.float().cpu().numpy()


def _case(et, seed, T, inn, out, std=0.05):
    x = et.synth.normal(seed, 1, (T, inn), 1.0)
    w = et.synth.normal(seed, 2, (out, inn), std)
    b = et.synth.normal(seed, 3, (out,), 0.1)
    return x, w, b


@pytest.mark.parametrize("bn", [0, 64, 128, 192, 256, 384])
@pytest.mark.parametrize("T,inn,out,act", [
    (128, 64, 128, 0), (256, 768, 768, 0), (2048, 768, 2304, 0), (512, 768, 3072, 2),
    (512, 3072, 768, 0), (100, 80, 48, 1), (1, 16, 16, 0), (333, 1024, 1008, 2),
])
def test_dense(et, orc, cuda, T, inn, out, act, bn):
    x, w, b = _case(et, 11, T, inn, out)
    et.lib().et_debug_force_gemm_bn(bn)
    try:
        y = et.linear_dense(_dev(x, cuda), _dev(w, cuda), _dev(b, cuda), act)
        assert et.device_error() == 0
    finally:
        et.lib().et_debug_force_gemm_bn(0)
    assert_close(_host(y), orc.linear_dense(x, w, b, act), f"dense {T}x{inn}x{out} bn{bn}",
                 dump=f"dense_{T}_{inn}_{out}_{bn}")


@pytest.mark.parametrize("pair_bn,persist", [(128, 0), (128, 1), (256, 0), (256, 1)])
@pytest.mark.parametrize("T,inn,out,act", [
    (256, 64, 256, 0), (2048, 768, 2304, 0), (512, 3072, 768, 0), (300, 768, 3072, 2),
    (1, 16, 16, 0), (333, 1008, 1008, 2), (4100, 272, 528, 1),
])
def test_dense_cta_pairs(et, orc, cuda, T, inn, out, act, pair_bn, persist):
    """The CTA-pair kernels (two SMs per 256-row tile) against the oracle, and bit for bit
    against the single-CTA kernels: ragged M, N and K, one and several tiles per pair."""
    import ctypes
    import torch
    x, w, b = _case(et, 13, T, inn, out)
    xd, wd, bd = _dev(x, cuda), _dev(w, cuda), _dev(b, cuda)
    L = et.lib()
    try:
        L.et_debug_force_gemm_pair(ctypes.c_int(0))
        y0 = et.linear_dense(xd, wd, bd, act)
        L.et_debug_force_gemm_pair(ctypes.c_int(pair_bn))
        L.et_debug_force_gemm_pair_persist(ctypes.c_int(persist))
        y = et.linear_dense(xd, wd, bd, act)
        assert et.device_error() == 0
    finally:
        L.et_debug_force_gemm_pair(ctypes.c_int(-1))
        L.et_debug_force_gemm_pair_persist(ctypes.c_int(-1))
    assert_close(_host(y), orc.linear_dense(x, w, b, act), f"pair {T}x{inn}x{out} bn{pair_bn}")
    assert torch.equal(y, y0), "CTA-pair and single-CTA results differ"


@pytest.mark.parametrize("bn", [128, 192, 256])
@pytest.mark.parametrize("T,inn,out,act", [
    (256, 64, 256, 0), (2048, 768, 3072, 2), (512, 3072, 768, 0), (300, 768, 3072, 2),
    (1, 16, 16, 0), (333, 1008, 1008, 2), (4100, 272, 528, 1),
])
def test_dense_256_row_tiles(et, orc, cuda, T, inn, out, act, bn):
    """The 256-row single-CTA tiles (two accumulators per weight tile) against the oracle and,
    bit for bit, against the 128-row kernels."""
    import ctypes
    import torch
    x, w, b = _case(et, 14, T, inn, out)
    xd, wd, bd = _dev(x, cuda), _dev(w, cuda), _dev(b, cuda)
    L = et.lib()
    try:
        L.et_debug_force_gemm_pair(ctypes.c_int(0))
        L.et_debug_force_gemm_tall(ctypes.c_int(0))
        y0 = et.linear_dense(xd, wd, bd, act)
        L.et_debug_force_gemm_tall(ctypes.c_int(bn))
        y = et.linear_dense(xd, wd, bd, act)
        assert et.device_error() == 0
    finally:
        L.et_debug_force_gemm_pair(ctypes.c_int(-1))
        L.et_debug_force_gemm_tall(ctypes.c_int(-1))
    assert_close(_host(y), orc.linear_dense(x, w, b, act), f"tall {T}x{inn}x{out} bn{bn}")
    assert torch.equal(y, y0), "256-row and 128-row tiles differ"


def test_dense_constant_closed_form(et, cuda):
    """W = 1, x = 1, b = 0.5 gives in + 0.5 everywhere (the reference's constant generators,
    Linear/gen_linear.hpp:15-23, Linear/test/test_tile.cu:61-74)."""
    import torch
    T, inn, out = 128, 256, 64
    x = torch.ones((T, inn), dtype=torch.float16, device=cuda)
    w = torch.ones((out, inn), dtype=torch.float16, device=cuda)
    b = torch.full((out,), 0.5, dtype=torch.float16, device=cuda)
    y = et.linear_dense(x, w, b)
    assert et.device_error() == 0
    assert torch.all(y.float() == inn + 0.5)


def test_dense_no_bias(et, orc, cuda):
    x, w, _ = _case(et, 12, 200, 128, 96)
    y = et.linear_dense(_dev(x, cuda), _dev(w, cuda), None, 0)
    assert_close(_host(y), orc.linear_dense(x, w, None, 0), "dense no bias")


@pytest.mark.parametrize("sparsity", [0.0, 0.5, 0.8, 0.95, 1.0])
@pytest.mark.parametrize("T,inn,out,act", [(256, 768, 768, 0), (300, 768, 3072, 2),
                                           (128, 3072, 768, 0), (64, 64, 48, 1)])
def test_tile(et, orc, cuda, T, inn, out, act, sparsity):
    x, w, b = _case(et, 21, T, inn, out)
    w = et.synth.prune_tiles(w, 21, 4, sparsity)
    rp, ro, tiles = et.synth.dense_to_tile(w)
    import ctypes
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    assert et.lib().et_validate_tile_mat(vp(rp), vp(ro) if len(ro) else None, len(ro), inn,
                                         out) == 0
    y = et.linear_tile(_dev(x, cuda), _dev(rp, cuda), _dev(ro, cuda) if len(ro) else None,
                       _dev(tiles, cuda) if len(ro) else None, out, _dev(b, cuda), act)
    assert et.device_error() == 0
    ref = orc.linear_tile(x, rp, ro, tiles.astype(np.float32), out, b, act)
    assert_close(_host(y), ref, f"tile {T}x{inn}x{out} s={sparsity}",
                 dump=f"tile_{T}_{inn}_{out}_{sparsity}")
    # format-native loop agrees with the dense evaluation of the densified weights
    assert_close(ref, orc.linear_dense(x, w, b, act), "oracle tile vs dense", 1e-5, 1e-4)
    # re-packed weights: same result bit for bit, and the packing is a pure permutation
    if len(ro):
        pk = et.PackedTiles(rp, ro, tiles, inn, out, cuda)
        import torch
        L = et.lib()
        # the packed-weight kernels (one item per CTA with one / two panels of 128 outputs, the
        # persistent form, the choice by shape) accumulate like the tile-CSR forward: same
        # result bit for bit
        for mode, wide in ((0, 0), (0, 1), (1, -1), (-1, -1)):
            L.et_debug_set_tile_persist(ctypes.c_int(mode))
            L.et_debug_set_tile_wide(ctypes.c_int(wide))
            try:
                yp = et.linear_tile_packed(_dev(x, cuda), pk, _dev(b, cuda), act)
                assert et.device_error() == 0
            finally:
                L.et_debug_set_tile_wide(ctypes.c_int(-1))
                L.et_debug_set_tile_persist(ctypes.c_int(-1))
            assert torch.equal(yp, y), f"packed (mode={mode}, wide={wide}) and tile-CSR forward differ"
        # the warp-level kernel (mma.sync, every warp walking its block row's tiles) sums in
        # another order
        if inn % 64 == 0:
            L.et_debug_set_tile_rows(ctypes.c_int(1))
            try:
                yr = et.linear_tile(_dev(x, cuda), _dev(rp, cuda), _dev(ro, cuda), _dev(tiles, cuda), out,
                                    _dev(b, cuda), act)
                assert et.device_error() == 0
            finally:
                L.et_debug_set_tile_rows(ctypes.c_int(0))
            assert_close(_host(yr), ref, f"tile (warp-level) {T}x{inn}x{out} s={sparsity}")
        assert np.array_equal(np.sort(pk.perm_host), np.arange(len(ro)))
        packed = pk.tiles.cpu().numpy().reshape(-1, 16, 2, 8)
        unsw = packed.copy()
        flip = ((np.arange(16) >> 2) & 1).astype(bool)
        unsw[:, flip] = packed[:, flip][:, :, ::-1]
        assert np.array_equal(unsw.reshape(-1, 256), tiles[pk.perm_host])
    # expansion to dense restores the pruned matrix exactly
    dense = et.tile_densify(_dev(rp, cuda), _dev(ro, cuda) if len(ro) else None,
                            _dev(tiles, cuda) if len(ro) else None, inn, out)
    assert np.array_equal(_host(dense), w)
    keep = 0.10 if out >= 3072 else (0.15 if out >= 2048 else 0.02)
    assert et.tile_prefer_dense(inn, out, len(ro)) == (len(ro) > keep * (inn // 16) * (out // 16))


def test_tile_empty_block_rows(et, orc, cuda):
    """Block rows without any tile receive the bias alone."""
    x, w, b = _case(et, 22, 160, 128, 256)
    w[16:48] = 0
    w[240:] = 0
    rp, ro, tiles = et.synth.dense_to_tile(w)
    y = et.linear_tile(_dev(x, cuda), _dev(rp, cuda), _dev(ro, cuda), _dev(tiles, cuda), 256,
                       _dev(b, cuda), 0)
    assert et.device_error() == 0
    assert_close(_host(y), orc.linear_dense(x, w, b, 0), "tile empty rows")


@pytest.mark.parametrize("T,inn,out", [(300, 256, 512), (2048, 768, 3072), (77, 64, 4096)])
@pytest.mark.parametrize("sparsity", [0.0, 0.5, 0.9])
def test_row(et, orc, cuda, sparsity, T, inn, out):
    """Row-pruned Linear: kept features computed compressed into the head of each output row,
    then spread in place (pruned columns receive act(bias)); the compressed form on its own."""
    import torch
    x, w, b = _case(et, 31, T, inn, out)
    row_id = et.synth.choose_ids(31, 5, out, sparsity)
    rid, rows = et.synth.dense_to_row(w, row_id)
    for act in (0, 2):
        y = et.linear_row(_dev(x, cuda), _dev(rid, cuda), _dev(rows, cuda), out, _dev(b, cuda), act)
        assert et.device_error() == 0
        assert_close(_host(y), orc.linear_row(x, rid, rows, out, b, act), f"row s={sparsity}")
    yc = et.linear_row_compressed(_dev(x, cuda), _dev(rid, cuda), _dev(rows, cuda), _dev(b, cuda))
    assert_close(_host(yc), orc.linear_row_compressed(x, rid, rows, b), "row compressed")
    # the spread output holds exactly the compressed values in the kept columns
    y0 = et.linear_row(_dev(x, cuda), _dev(rid, cuda), _dev(rows, cuda), out, _dev(b, cuda), 0)
    assert torch.equal(y0[:, torch.from_numpy(rid.astype(np.int64)).to(cuda)], yc)


def test_row_kept_count_not_a_multiple_of_8(et, orc, cuda):
    """A kept list the 16-byte stores cannot serve takes the fill + scatter path."""
    T, inn, out = 130, 128, 256
    x, w, b = _case(et, 32, T, inn, out)
    row_id = et.synth.choose_ids(32, 5, out, 0.5)[:-3]
    rid, rows = et.synth.dense_to_row(w, row_id)
    y = et.linear_row(_dev(x, cuda), _dev(rid, cuda), _dev(rows, cuda), out, _dev(b, cuda), 2)
    assert et.device_error() == 0
    assert_close(_host(y), orc.linear_row(x, rid, rows, out, b, 2), "row, 125 kept")


@pytest.mark.parametrize("T,inn,out", [(260, 512, 256),      # a row of X fits a shared-memory line
                                       (40, 16384, 64)])      # it does not: direct gather
@pytest.mark.parametrize("sparsity", [0.0, 0.5, 0.9])
def test_col(et, orc, cuda, sparsity, T, inn, out):
    x, w, b = _case(et, 41, T, inn, out)
    col_id = et.synth.choose_ids(41, 5, inn, sparsity)
    cid, cols = et.synth.dense_to_col(w, col_id)
    y = et.linear_col(_dev(x, cuda), _dev(cid, cuda), _dev(cols, cuda), _dev(b, cuda), 1)
    assert et.device_error() == 0
    assert_close(_host(y), orc.linear_col(x, cid, cols, b, 1), f"col s={sparsity}")


@pytest.mark.parametrize("sparsity", [0.0, 0.9, 1.0])
def test_1x16(et, orc, cuda, sparsity):
    T, inn, out = 200, 256, 128
    x, w, b = _case(et, 51, T, inn, out)
    w = et.synth.prune_1x16(w, 51, 6, sparsity)
    ti, ri, data = et.synth.dense_to_1x16(w)
    y = et.linear_1x16(_dev(x, cuda), _dev(ti, cuda), _dev(ri, cuda) if len(ri) else None,
                       _dev(data, cuda) if len(ri) else None, out, _dev(b, cuda), 2)
    assert et.device_error() == 0
    assert_close(_host(y), orc.linear_1x16(x, ti, ri, data, out, b, 2), f"1x16 s={sparsity}")


@pytest.mark.parametrize("sparsity", [0.5, 0.95])
def test_csr(et, orc, cuda, sparsity):
    T, inn, out = 100, 256, 200
    x, w, b = _case(et, 61, T, inn, out)
    keep = et.synth.keep_exact(61, 7, out * inn, sparsity).reshape(out, inn)
    w = w * keep
    ip, ix, data = et.synth.dense_to_csr(w)
    y = et.linear_csr(_dev(x, cuda), _dev(ip, cuda), _dev(ix, cuda), _dev(data, cuda), out,
                      _dev(b, cuda), 0)
    assert et.device_error() == 0
    assert_close(_host(y), orc.linear_csr(x, ip, ix, data, out, b, 0), f"csr s={sparsity}")


def test_bad_arguments_are_rejected_before_launch(et, cuda):
    """Host-side failure injection: bad shapes / pointers return a status, nothing launches."""
    import torch
    x = torch.zeros((16, 24), dtype=torch.float16, device=cuda)
    w = torch.zeros((16, 24), dtype=torch.float16, device=cuda)
    with pytest.raises(et.EtError):
        et.linear_dense(x, w)  # in % 16 != 0
    x = torch.zeros((16, 32), dtype=torch.float16, device=cuda)
    w = torch.zeros((16, 32), dtype=torch.float16, device=cuda)
    import ctypes
    vp = ctypes.c_void_p
    st = et.lib().et_linear_dense_fwd(None, vp(w.data_ptr()), None, vp(x.data_ptr()), 16, 32, 16, 0,
                                      None)
    assert st == -1
    st = et.lib().et_linear_dense_fwd(vp(x.data_ptr() + 2), vp(w.data_ptr()), None,
                                      vp(x.data_ptr()), 16, 32, 16, 0, None)
    assert st == -2
    assert et.device_error() == 0


def test_dense_plan_sweep(et, orc, cuda):
    """Shapes chosen to hit every branch of the tile plan (single-tile CTAs, persistent 128 / 192
    / 256-wide tiles, CTA pairs of both widths) with ragged edges, through the automatic
    dispatch, against the oracle."""
    shapes = [
        (2048, 768, 3072, 2),   # persistent 192-wide tiles
        (2048, 3072, 768, 0),   # 256 x 128 CTA pairs (long K, few tiles)
        (2048, 1024, 4096, 1),  # 256 x 256 CTA pairs
        (2064, 784, 2320, 0),   # single-tile CTAs, every dimension ragged
        (4104, 272, 3088, 2),   # many tiles, ragged
        (130, 2048, 144, 0),    # long K, one tile column, M just above one tile
        (255, 4096, 4096, 1),   # M below the pair threshold
        (257, 2064, 528, 0),    # M just above it, pair tiles half empty
        (24, 48, 48, 2),        # everything smaller than one tile
    ]
    for i, (T, inn, out, act) in enumerate(shapes):
        x, w, b = _case(et, 300 + i, T, inn, out)
        y = et.linear_dense(_dev(x, cuda), _dev(w, cuda), _dev(b, cuda), act)
        assert et.device_error() == 0
        assert_close(_host(y), orc.linear_dense(x, w, b, act), f"plan sweep {T}x{inn}x{out} act{act}")
