"""GPU parity of the fused attention kernel against the oracle: sequence lengths from the
reference's sweep (test/Attention/test_seqlen.cu: 16..512), all mask kinds, fused-QKV layout,
pruned Q/K head width (48), ragged lengths, batch > 1."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _qkv(et, seed, batch, seq, nhead, dh_qk, dh_v, std=1.0):
    T = batch * seq
    q = et.synth.normal(seed, 1, (T, nhead * dh_qk), std)
    k = et.synth.normal(seed, 2, (T, nhead * dh_qk), std)
    v = et.synth.normal(seed, 3, (T, nhead * dh_v), std)
    return q, k, v


@pytest.mark.parametrize("batch,seq,nhead,dh_qk,dh_v", [
    (1, 128, 1, 64, 64), (2, 128, 12, 64, 64), (1, 16, 2, 16, 16), (3, 48, 2, 32, 64),
    (2, 256, 4, 64, 64), (1, 384, 2, 64, 64), (1, 512, 3, 64, 64), (2, 200, 2, 48, 64),
    (1, 1000, 1, 64, 64), (1, 128, 2, 128, 128), (1, 300, 1, 96, 112), (1, 4096, 2, 64, 64),
])
@pytest.mark.parametrize("mask_kind", [0, 1])
def test_attention(et, orc, cuda, batch, seq, nhead, dh_qk, dh_v, mask_kind):
    q, k, v = _qkv(et, 100 + seq, batch, seq, nhead, dh_qk, dh_v)
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh_qk, dh_v,
                     mask_kind)
    assert et.device_error() == 0
    ref = orc.attention(q, k, v, batch, seq, nhead, dh_qk, dh_v, mask_kind)
    assert_close(z.float().cpu().numpy(), ref, f"attention b{batch} s{seq} h{nhead} m{mask_kind}",
                 dump=f"attn_{batch}_{seq}_{nhead}_{dh_qk}_{dh_v}_{mask_kind}")


def test_attention_uniform_scores_return_mean_of_v(et, cuda):
    """Constant Q and K give uniform probabilities: Z = mean of V rows (closed form implied
    by the reference's constant-input drivers)."""
    import torch
    batch, seq, nhead, dh = 1, 128, 2, 64
    q = torch.full((seq, nhead * dh), 0.25, dtype=torch.float16, device=cuda)
    v = _dev(et.synth.normal(9, 1, (seq, nhead * dh), 1.0), cuda)
    z = et.attention(q, q, v, batch, seq, nhead, dh, dh)
    ref = v.float().mean(dim=0, keepdim=True).expand(seq, -1)
    assert torch.allclose(z.float(), ref, atol=3e-3)


def test_attention_fused_qkv_layout(et, orc, cuda):
    """Q, K, V as column ranges of one [T, 2*kdim + vdim] buffer (Attention.h:258-263)."""
    batch, seq, nhead, dh = 2, 128, 4, 64
    kdim = vdim = nhead * dh
    buf = et.synth.normal(77, 1, (batch * seq, 2 * kdim + vdim), 1.0)
    d = _dev(buf, cuda)
    z = et.attention(d[:, :kdim], d[:, kdim:2 * kdim], d[:, 2 * kdim:], batch, seq, nhead, dh, dh)
    assert et.device_error() == 0
    ref = orc.attention(buf[:, :kdim], buf[:, kdim:2 * kdim], buf[:, 2 * kdim:], batch, seq, nhead,
                        dh, dh)
    assert_close(z.float().cpu().numpy(), ref, "fused qkv layout")


@pytest.mark.parametrize("seq", [128, 384])
def test_attention_padding_mask(et, orc, cuda, seq):
    batch, nhead, dh = 4, 2, 64
    q, k, v = _qkv(et, 55, batch, seq, nhead, dh, dh)
    vl = np.array([seq, seq // 3, 1, 130 if seq > 130 else 17], dtype=np.int32)
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh, dh, 2,
                     None, _dev(vl, cuda))
    assert et.device_error() == 0
    ref = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 2, None, vl)
    assert_close(z.float().cpu().numpy(), ref, "padding mask")


def test_attention_zero_valid_length_gives_zeros(et, cuda):
    import torch
    batch, seq, nhead, dh = 2, 64, 1, 32
    q = _dev(et.synth.normal(3, 1, (batch * seq, dh), 1.0), cuda)
    vl = _dev(np.array([0, seq], dtype=np.int32), cuda)
    z = et.attention(q, q, q, batch, seq, nhead, dh, dh, 2, None, vl)
    assert et.device_error() == 0
    assert torch.all(z[:seq] == 0)
    assert torch.isfinite(z.float()).all()


@pytest.mark.parametrize("seq", [64, 128, 272])
def test_attention_additive_mask(et, orc, cuda, seq):
    """General additive [seq, seq] mask; the causal one of Attention.h:97-104 must agree with
    ET_MASK_CAUSAL."""
    batch, nhead, dh = 2, 2, 64
    q, k, v = _qkv(et, 66, batch, seq, nhead, dh, dh)
    causal = np.where(np.tril(np.ones((seq, seq), bool)), 0.0, -np.inf).astype(np.float16)
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh, dh, 3,
                     _dev(causal, cuda))
    assert et.device_error() == 0
    ref = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 1)
    assert_close(z.float().cpu().numpy(), ref, "additive causal")
    soft = et.synth.normal(67, 9, (seq, seq), 1.0)
    soft[3, :] = -np.inf  # one fully dropped query row -> zeros
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh, dh, 3,
                     _dev(soft, cuda))
    ref = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 3, soft.astype(np.float32))
    assert_close(z.float().cpu().numpy(), ref, "additive soft")


def test_attention_is_deterministic(et, cuda):
    import torch
    q, k, v = _qkv(et, 88, 2, 256, 4, 64, 64)
    a = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), 2, 256, 4, 64, 64, 1)
    b = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), 2, 256, 4, 64, 64, 1)
    assert torch.equal(a, b)


@pytest.mark.parametrize("batch,seq,nhead,dh,sparsity", [
    (2, 128, 4, 64, 0.5), (1, 200, 12, 64, 0.3), (2, 64, 2, 32, 0.75), (1, 300, 3, 128, 0.5),
])
@pytest.mark.parametrize("mask_kind", [0, 1])
def test_attention_pruned_v(et, orc, cuda, batch, seq, nhead, dh, sparsity, mask_kind):
    """V arrives column-compressed (the output of a row-pruned V projection); Z is written in
    full with zeros at pruned features (Attention/kernels.cu:425-459 + the missing store)."""
    T, vdim = batch * seq, nhead * dh
    q, k, v = _qkv(et, 300 + seq, batch, seq, nhead, dh, dh)
    col_id = et.synth.choose_ids(301, 5, vdim, sparsity, multiple=8)
    if seq == 64:  # leave one head without any kept feature
        col_id = col_id[col_id >= dh]
        col_id = col_id[: len(col_id) // 8 * 8]
    hp = et.synth.head_ptr_for(col_id, nhead, vdim)
    vc = np.ascontiguousarray(v[:, col_id])
    z = et.attention_pruned_v(_dev(q, cuda), _dev(k, cuda), _dev(vc, cuda), _dev(col_id, cuda),
                              _dev(hp, cuda), batch, seq, nhead, dh, dh, mask_kind)
    assert et.device_error() == 0
    ref = orc.attention_pruned_v(q, k, vc, col_id, hp, batch, seq, nhead, dh, dh, mask_kind)
    assert_close(z.float().cpu().numpy(), ref, f"pruned V s{seq} h{nhead}",
                 dump=f"prunedv_{seq}_{nhead}_{mask_kind}")
    pruned = np.setdiff1d(np.arange(vdim), col_id)
    assert np.all(z.float().cpu().numpy()[:, pruned] == 0)


@pytest.mark.parametrize("batch,seq,nhead,dh,emdim", [
    (2, 128, 4, 64, 256), (1, 128, 12, 64, 768), (2, 96, 2, 32, 80), (1, 300, 3, 64, 320),
    (1, 512, 2, 64, 256),
])
@pytest.mark.parametrize("mask_kind", [0, 1])
def test_fused_vo_attention(et, orc, cuda, batch, seq, nhead, dh, emdim, mask_kind):
    """out = sum_h P_h (X W_vo,h + b_h) + b_o (Fused_attention.cu:94-115, Linear_VO.h:38-58)."""
    T = batch * seq
    q = et.synth.normal(400 + seq, 1, (T, nhead * dh), 1.0)
    k = et.synth.normal(400 + seq, 2, (T, nhead * dh), 1.0)
    x = et.synth.normal(400 + seq, 3, (T, emdim), 1.0)
    wvo = et.synth.normal(400 + seq, 4, (nhead, emdim, emdim), 0.05)
    bvo = et.synth.normal(400 + seq, 5, (nhead, emdim), 0.05)
    bo = et.synth.normal(400 + seq, 6, (emdim,), 0.1)
    vo = et.linear_vo(_dev(x, cuda), _dev(wvo, cuda), _dev(bvo, cuda), batch, seq, nhead, emdim)
    assert et.device_error() == 0
    # VO[b][h] = X_b W_vo[h] + b[h]
    xf = x.astype(np.float32).reshape(batch, seq, emdim)
    vo_ref = np.einsum("bse,heo->bhso", xf, wvo.astype(np.float32)) + \
        bvo.astype(np.float32)[None, :, None, :]
    assert_close(vo.float().cpu().numpy(), vo_ref.reshape(-1, emdim), "linear_vo",
                 dump=f"linvo_{seq}_{emdim}")
    out = et.fused_vo_attention(_dev(q, cuda), _dev(k, cuda), vo, _dev(bo, cuda), batch, seq,
                                nhead, dh, emdim, mask_kind)
    assert et.device_error() == 0
    vo16 = vo.float().cpu().numpy()
    ref = orc.fused_vo_attention(q, k, vo16, bo, batch, seq, nhead, dh, emdim, mask_kind)
    assert_close(out.float().cpu().numpy(), ref, f"fused VO s{seq} e{emdim}",
                 dump=f"fusedvo_{seq}_{emdim}_{mask_kind}")
    out2 = et.fused_vo_attention(_dev(q, cuda), _dev(k, cuda), vo, _dev(bo, cuda), batch, seq,
                                 nhead, dh, emdim, mask_kind)
    import ctypes
    import torch
    assert torch.equal(out, out2), "head reduction must be deterministic"
    # every width of the output chunk a CTA owns gives the same bits (heads are reduced in the
    # same order inside every accumulator column)
    L = et.lib()
    try:
        for nc in (64, 128, 256):
            L.et_debug_set_vo_chunk(ctypes.c_int(nc))
            o = et.fused_vo_attention(_dev(q, cuda), _dev(k, cuda), vo, _dev(bo, cuda), batch, seq,
                                      nhead, dh, emdim, mask_kind)
            assert et.device_error() == 0
            assert torch.equal(out, o), f"chunk width {nc}"
    finally:
        L.et_debug_set_vo_chunk(ctypes.c_int(0))


@pytest.mark.parametrize("batch,seq,nhead,dh,em,mask_kind,sparsity", [
    (1, 128, 12, 64, 768, 0, 0.8),    # the reference's own shape: one sequence, BERT-base heads
    (2, 128, 4, 64, 256, 1, 0.6),
    (3, 100, 4, 64, 256, 2, 0.6),     # token blocks of the projection span two sequences
    (9, 16, 2, 32, 64, 0, 0.5),       # eight sequences per token block; heads narrower than a TMA box
    (4, 512, 12, 64, 768, 1, 0.8),    # several query blocks per sequence, causal
    (40, 128, 12, 64, 768, 2, 0.9),   # more pieces of work than CTAs
    (2, 200, 3, 48, 144, 3, 0.5),     # ragged blocks, additive mask, 48-wide heads
    (1, 128, 2, 64, 128, 0, 0.97),    # output block rows without any stored tile
])
def test_attention_fuse_o(et, orc, cuda, batch, seq, nhead, dh, em, mask_kind, sparsity):
    """Attention and the tile-CSR output projection (kernel_fuseO.cu) as one kernel and as two
    chained kernels: against the oracle, and bit for bit against each other."""
    import torch
    q, k, v = _qkv(et, 500 + seq, batch, seq, nhead, dh, dh)
    wo = et.synth.prune_tiles(et.synth.normal(500, 4, (em, nhead * dh), 0.05), 500, 5, sparsity)
    bo = et.synth.normal(500, 6, (em,), 0.1)
    rp, ro, tiles = et.synth.dense_to_tile(wo)
    vl = np.array([(37 * i + 5) % seq + 1 for i in range(batch)], dtype=np.int32)
    mask = None
    if mask_kind == 3:
        mask = np.where(et.synth.normal(500, 7, (seq, seq), 1.0).astype(np.float32) > 0.8,
                        -np.inf, 0.0).astype(np.float16)
        mask[np.arange(seq), np.arange(seq)] = 0
    d = lambda a: None if a is None else _dev(a, cuda)
    args = (d(q), d(k), d(v), d(rp), d(ro), d(tiles), d(bo), batch, seq, nhead, dh, dh, em,
            mask_kind, d(mask), d(vl) if mask_kind == 2 else None)
    out = et.attention_fuse_o(*args, single_launch=True)
    assert et.device_error() == 0
    again = et.attention_fuse_o(*args, single_launch=True)  # the counters are zero again after a call
    assert et.device_error() == 0
    two = et.attention_fuse_o(*args)
    assert et.device_error() == 0
    assert torch.equal(out, two), "one kernel and two kernels must agree bit for bit"
    assert torch.equal(out, again)
    z = orc.round_fp16(orc.attention(q, k, v, batch, seq, nhead, dh, dh, mask_kind, mask,
                                     vl if mask_kind == 2 else None))
    assert_close(out.float().cpu().numpy(), orc.linear_dense(z, wo, bo),
                 f"attention + tile O b{batch} s{seq} m{mask_kind}")


def test_attention_fuse_o_work_order(et, cuda):
    """The one-kernel form's per-ticket trace (test hook): every piece of work ran once, and no
    projection item finished before the attention units whose rows it reads."""
    import ctypes
    import torch
    batch, seq, nhead, dh, em = 24, 128, 12, 64, 768
    q, k, v = _qkv(et, 640, batch, seq, nhead, dh, dh)
    wo = et.synth.prune_tiles(et.synth.normal(640, 4, (em, nhead * dh), 0.05), 640, 5, 0.8)
    rp, ro, tiles = et.synth.dense_to_tile(wo)
    n_att, npanel = batch * nhead, em // 128
    n_items = npanel * batch
    trace = torch.zeros((n_att + n_items, 4), dtype=torch.int64, device=cuda)
    L = et.lib()
    L.et_debug_set_fuse_o_trace(ctypes.c_void_p(trace.data_ptr()))
    try:
        et.attention_fuse_o(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), _dev(rp, cuda), _dev(ro, cuda),
                            _dev(tiles, cuda), None, batch, seq, nhead, dh, dh, em, 0,
                            single_launch=True)
        torch.cuda.synchronize()
    finally:
        L.et_debug_set_fuse_o_trace(ctypes.c_void_p(0))
    assert et.device_error() == 0
    t = trace.cpu().numpy()
    assert (t[:, 0] > 0).all() and (t[:, 1] >= t[:, 0]).all(), "a piece of work left no record"
    att_end = t[:n_att, 1].reshape(batch, nhead).max(axis=1)   # ticket = sequence * nhead + head
    item_end = t[n_att:, 1].reshape(batch, npanel)             # item = token block * npanel + panel
    assert (item_end > att_end[:, None]).all()


@pytest.mark.parametrize("batch,seq,hidden,nhead", [
    (2, 128, 768, 12), (3, 100, 256, 4), (1, 16, 64, 1), (16, 128, 768, 12), (2, 72, 208, 2),
])
@pytest.mark.parametrize("mask_kind", [0, 1, 2, 3])
def test_qkv_attention_fused(et, orc, cuda, batch, seq, hidden, nhead, mask_kind):
    """Projection + attention in one kernel against the oracle's Linear followed by its
    attention, for every mask kind, ragged sequence lengths and hidden sizes that are not a
    multiple of the 64-feature K block."""
    import torch
    T, kdim = batch * seq, nhead * 64
    x = et.synth.normal(600 + seq, 1, (T, hidden), 1.0)
    w = et.synth.normal(600 + seq, 2, (3 * kdim, hidden), 0.06)
    bq = et.synth.normal(600 + seq, 3, (3 * kdim,), 0.1)
    vl = np.array([(37 * i + 5) % seq + 1 for i in range(batch)], dtype=np.int32)
    if batch > 1:
        vl[1] = seq
    mask = None
    if mask_kind == 3:
        mask = np.where(et.synth.normal(600 + seq, 4, (seq, seq), 1.0).astype(np.float32) > 0.8,
                        -np.inf, 0.0).astype(np.float16)
        mask[np.arange(seq), np.arange(seq)] = 0
    d = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    z = et.qkv_attention(d(x), d(w), d(bq), batch, seq, nhead, kdim, kdim, mask_kind, d(mask),
                         d(vl) if mask_kind == 2 else None)
    assert et.device_error() == 0
    qkv = orc.round_fp16(orc.linear_dense(x, w, bq, 0))
    ref = orc.attention(qkv[:, :kdim], qkv[:, kdim:2 * kdim], qkv[:, 2 * kdim:], batch, seq, nhead,
                        64, 64, mask_kind, mask, vl if mask_kind == 2 else None)
    assert_close(z.float().cpu().numpy(), ref, f"fused qkv attention b{batch} s{seq} m{mask_kind}")
    # the separate kernels give the same result up to rounding
    q2 = et.linear_dense(d(x), d(w), d(bq))
    z2 = et.attention(q2[:, :kdim], q2[:, kdim:2 * kdim], q2[:, 2 * kdim:], batch, seq, nhead, 64,
                      64, mask_kind, d(mask), d(vl) if mask_kind == 2 else None)
    assert_close(z.float().cpu().numpy(), z2.float().cpu().numpy(), "fused vs separate kernels",
                 rel_tol=2e-3, abs_tol=4e-3)


def test_qkv_attention_rejects_other_shapes(et, cuda):
    import torch
    x = torch.zeros((256, 64), dtype=torch.float16, device=cuda)
    w = torch.zeros((192, 64), dtype=torch.float16, device=cuda)
    with pytest.raises(et.EtError):
        et.qkv_attention(x, w, None, 1, 256, 1, 64, 64)       # seq > 128
    w2 = torch.zeros((96, 64), dtype=torch.float16, device=cuda)
    with pytest.raises(et.EtError):
        et.qkv_attention(x[:128], w2, None, 1, 128, 1, 32, 32)  # 32-wide head


@pytest.mark.parametrize("batch,seq,nhead,dh,emdim,sparsity", [
    (2, 128, 4, 64, 256, 0.5), (1, 200, 3, 64, 320, 0.75), (2, 96, 2, 32, 80, 0.0),
])
def test_fused_vo_attention_column_pruned(et, orc, cuda, batch, seq, nhead, dh, emdim, sparsity):
    """Column-pruned V.O: projection and attention run at the kept width, the result is
    scattered back; pruned output features carry the bias alone."""
    T = batch * seq
    q = et.synth.normal(700 + seq, 1, (T, nhead * dh), 1.0)
    k = et.synth.normal(700 + seq, 2, (T, nhead * dh), 1.0)
    x = et.synth.normal(700 + seq, 3, (T, emdim), 1.0)
    wvo = et.synth.normal(700 + seq, 4, (nhead, emdim, emdim), 0.05)
    bvo = et.synth.normal(700 + seq, 5, (nhead, emdim), 0.05)
    bo = et.synth.normal(700 + seq, 6, (emdim,), 0.1)
    cid = et.synth.choose_ids(700 + seq, 7, emdim, sparsity)
    wc = np.ascontiguousarray(wvo[:, :, cid])
    bc = np.ascontiguousarray(bvo[:, cid])
    voc = et.linear_vo_pruned(_dev(x, cuda), _dev(wc, cuda), _dev(bc, cuda), batch, seq, nhead, emdim)
    assert et.device_error() == 0
    xf = x.astype(np.float32).reshape(batch, seq, emdim)
    vo_ref = np.einsum("bse,heo->bhso", xf, wc.astype(np.float32)) + bc.astype(np.float32)[None, :, None, :]
    assert_close(voc.float().cpu().numpy(), vo_ref.reshape(-1, len(cid)), "linear_vo_pruned")
    out = et.fused_vo_attention_pruned(_dev(q, cuda), _dev(k, cuda), voc, _dev(cid, cuda), _dev(bo, cuda),
                                       batch, seq, nhead, dh, emdim, 1)
    assert et.device_error() == 0
    comp = orc.fused_vo_attention(q, k, voc.float().cpu().numpy(), None, batch, seq, nhead, dh,
                                  len(cid), 1)
    ref = np.tile(bo.astype(np.float32), (T, 1))
    ref[:, cid] += orc.round_fp16(comp)
    assert_close(out.float().cpu().numpy(), ref, f"pruned fused VO s{seq} e{emdim}")
    pruned = np.setdiff1d(np.arange(emdim), cid)
    if len(pruned):
        assert np.array_equal(out.float().cpu().numpy()[:, pruned],
                              np.tile(bo.astype(np.float32)[pruned], (T, 1)))


def test_qkv_attention_edge_lengths(et, orc, cuda):
    """One-token sequences, a sequence whose valid length is zero (zeros out), no bias."""
    import torch
    d = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    hidden, nhead, kdim = 64, 1, 64
    w = et.synth.normal(810, 2, (3 * kdim, hidden), 0.1)
    # seq = 1: softmax over one key is 1, so Z = V
    x = et.synth.normal(810, 1, (5, hidden), 1.0)
    z = et.qkv_attention(d(x), d(w), None, 5, 1, nhead, kdim, kdim)
    assert et.device_error() == 0
    v = orc.round_fp16(orc.linear_dense(x, w[2 * kdim:], None, 0))
    assert_close(z.float().cpu().numpy(), v, "seq 1: Z equals V")
    # padding mask with an empty sequence
    batch, seq = 3, 40
    x = et.synth.normal(811, 1, (batch * seq, hidden), 1.0)
    vl = np.array([40, 0, 17], dtype=np.int32)
    z = et.qkv_attention(d(x), d(w), None, batch, seq, nhead, kdim, kdim, 2, None, d(vl))
    assert et.device_error() == 0
    zz = z.float().cpu().numpy()
    assert np.all(zz[seq:2 * seq] == 0)
    qkv = orc.round_fp16(orc.linear_dense(x, w, None, 0))
    ref = orc.attention(qkv[:, :kdim], qkv[:, kdim:2 * kdim], qkv[:, 2 * kdim:], batch, seq, nhead, 64,
                        64, 2, None, vl)
    assert_close(zz, ref, "padding with an empty sequence")
