"""Python harness over the C ABI of libet_b200.so (include/et_b200.h).

PyTorch is used only to own device memory and streams; every computation goes through the
C ABI with raw device pointers.  There is no fallback: if the CUDA library is missing or a
call reports an error, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_size_t, c_void_p

from . import sharding, synth, weights  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
# ET_B200_TEST_HOOKS=1 selects the build that also exports the et_debug_* test hooks (forced
# kernel plans, instruction-rate probes); the product library has none of them.
LIB_PATH = os.path.join(_HERE, "libet_b200_hooks.so" if os.environ.get("ET_B200_TEST_HOOKS") == "1"
                        else "libet_b200.so")

ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2
MASK_NONE, MASK_CAUSAL, MASK_PADDING, MASK_ADDITIVE = 0, 1, 2, 3
FMT_DENSE, FMT_TILE, FMT_TILE_PACKED, FMT_1X16, FMT_ROW, FMT_COL, FMT_CSR = range(7)

# Every symbol include/et_b200.h declares (checked by the CPU test-suite against the header).
ABI_SYMBOLS = [
    "et_status_string", "et_version", "et_built_for_sm", "et_device_error", "et_launch_count",
    "et_linear_dense_fwd", "et_linear_skip_layernorm_fwd", "et_linear_skip_layernorm_pays", "et_linear_tile_fwd", "et_tile_pack_dims", "et_tile_pack_plan",
    "et_tile_pack_tiles", "et_linear_tile_packed_fwd", "et_tile_prefer_dense", "et_tile_densify",
    "et_linear_row_fwd", "et_encoder_ffn_fwd", "et_peer_buffer_bytes", "et_peer_buffer_create",
    "et_peer_buffer_open", "et_peer_buffer_close", "et_peer_buffer_destroy", "et_peer_buffer_y",
    "et_peer_buffer_partial", "et_hp_signal_partial_fwd", "et_hp_reduce_layernorm_fwd", "et_hp_wait_fwd", "et_peer_buffer_out", "et_hp_allgather_rows_fwd",
    "et_linear_row_compressed_fwd", "et_linear_col_fwd", "et_linear_col_noalloc_fwd",
    "et_linear_1x16_fwd", "et_1x16_prefer_dense", "et_1x16_densify",
    "et_linear_csr_fwd", "et_validate_tile_mat", "et_validate_id_list", "et_validate_1x16",
    "et_validate_csr", "et_skip_layernorm_fwd", "et_layernorm_fwd", "et_act_fwd",
    "et_bias_add_fwd", "et_attention_fwd", "et_qkv_attention_fwd", "et_attention_pruned_v_fwd",
    "et_linear_vo_pruned_fwd", "et_fused_vo_attention_pruned_fwd",
    "et_attention_fuse_o_fwd", "et_attention_fuse_o_single_launch_fwd",
    "et_fused_vo_attention_fwd", "et_linear_vo_fwd",
    "et_encoder_layer_workspace_bytes", "et_encoder_layer_fwd",
    "et_attention_units_fwd", "et_encoder_attention_units_fwd", "et_encoder_after_attention_fwd",
]


class EtError(RuntimeError):
    pass


class LinearDesc(ctypes.Structure):
    """et_linear_t"""
    _fields_ = [("format", c_int), ("in_", c_int), ("out", c_int), ("weight", c_void_p),
                ("row_ptr", c_void_p), ("row_off", c_void_p), ("nnz_tiles", c_int),
                ("bias", c_void_p), ("pk_mask", c_void_p), ("pk_off", c_void_p)]


class EncoderLayerDesc(ctypes.Structure):
    """et_encoder_layer_t"""
    _fields_ = [("qkv", LinearDesc), ("o", LinearDesc), ("ffn1", LinearDesc), ("ffn2", LinearDesc),
                ("ln1_gamma", c_void_p), ("ln1_beta", c_void_p), ("ln2_gamma", c_void_p),
                ("ln2_beta", c_void_p), ("hidden", c_int), ("nhead", c_int), ("kdim", c_int),
                ("vdim", c_int), ("ff", c_int), ("act", c_int)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the CUDA library; raises if it has not been built (no CPU fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EtError(f"{LIB_PATH} is missing: run `python scpaper-2021_b200/build.py` "
                          "(the library has no CPU fallback)")
        L = ctypes.CDLL(LIB_PATH)
        L.et_status_string.restype = ctypes.c_char_p
        L.et_status_string.argtypes = [c_int]
        L.et_launch_count.restype = ctypes.c_longlong
        L.et_encoder_layer_workspace_bytes.restype = c_size_t
        L.et_encoder_layer_workspace_bytes.argtypes = [c_void_p, c_int, c_int]
        _lib = L
    return _lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        raise EtError(f"{what}: status {status} ({lib().et_status_string(status).decode()})")


def device_error() -> int:
    """Synchronises and returns (then clears) the device error word; 0 = no kernel complained."""
    code = c_int(0)
    check(lib().et_device_error(ctypes.byref(code)), "et_device_error")
    return code.value


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _empty(shape, like):
    import torch
    return torch.empty(shape, dtype=torch.float16, device=like.device)


# ---- Linear layers ------------------------------------------------------------------------

def linear_dense(x, w, bias=None, act=ACT_NONE, out=None):
    """`out`: optional preallocated [T, out] result (no allocation inside the call)."""
    T, inn = x.shape
    y = _empty((T, w.shape[0]), x) if out is None else out
    out = w.shape[0]
    check(lib().et_linear_dense_fwd(_p(x), _p(w), _p(bias), _p(y), c_int(T), c_int(inn),
                                    c_int(out), c_int(act), _stream()), "et_linear_dense_fwd")
    return y


def linear_tile(x, row_ptr, row_off, tiles, out, bias=None, act=ACT_NONE):
    T, inn = x.shape
    y = _empty((T, out), x)
    nnz = int(tiles.shape[0]) if tiles is not None else 0
    check(lib().et_linear_tile_fwd(_p(row_ptr), _p(row_off) if nnz else None,
                                   _p(tiles) if nnz else None, c_int(nnz), _p(bias), _p(x), _p(y),
                                   c_int(T), c_int(inn), c_int(out), c_int(act), _stream()),
          "et_linear_tile_fwd")
    return y


class PackedTiles:
    """Tile-CSR weights re-packed for et_linear_tile_packed_fwd.  Built from host arrays
    (row_ptr, row_off, tiles[nnz, 256] fp16): the plan runs on the host, the tiles are
    permuted on the GPU."""

    def __init__(self, row_ptr, row_off, tiles, inn: int, out: int, device="cuda"):
        import numpy as np
        import torch
        nnz = int(tiles.shape[0])
        npanel, nchunk = c_int(0), c_int(0)
        check(lib().et_tile_pack_dims(c_int(inn), c_int(out), ctypes.byref(npanel),
                                      ctypes.byref(nchunk)), "et_tile_pack_dims")
        n = npanel.value * nchunk.value
        rp = np.ascontiguousarray(row_ptr, np.int32)
        ro = np.ascontiguousarray(row_off, np.int32)
        mask = np.zeros(n, np.uint32)
        off = np.zeros(n, np.int32)
        perm = np.zeros(max(nnz, 1), np.int32)
        vp = lambda a: a.ctypes.data_as(c_void_p)
        check(lib().et_tile_pack_plan(vp(rp), vp(ro) if nnz else None, c_int(nnz), c_int(inn),
                                      c_int(out), vp(mask), vp(off), vp(perm)), "et_tile_pack_plan")
        self.inn, self.out, self.nnz = inn, out, nnz
        self.perm_host = perm[:nnz].copy()
        self.row_ptr = torch.from_numpy(rp).to(device)
        self.pk_mask = torch.from_numpy(mask.view(np.int32)).to(device)
        self.pk_off = torch.from_numpy(off).to(device)
        self.tiles = torch.empty((max(nnz, 1), 256), dtype=torch.float16, device=device)
        if nnz:
            src = torch.from_numpy(np.ascontiguousarray(tiles)).to(device)
            dperm = torch.from_numpy(self.perm_host).to(device)
            check(lib().et_tile_pack_tiles(_p(src), _p(dperm), c_int(nnz), _p(self.tiles),
                                           _stream()), "et_tile_pack_tiles")
            torch.cuda.current_stream().synchronize()


def tile_prefer_dense(inn: int, out: int, nnz_tiles: int) -> bool:
    """Plan-time choice: True when the dense GEMM on the expanded weight is expected to beat
    the tile kernel on B200."""
    return bool(lib().et_tile_prefer_dense(c_int(inn), c_int(out), c_int(nnz_tiles)))


def tile_densify(row_ptr, row_off, tiles, inn: int, out: int):
    """dense[out, in] fp16 from device tile-CSR arrays (pruned tiles zero)."""
    import torch
    dense = torch.empty((out, inn), dtype=torch.float16, device=row_ptr.device)
    nnz = 0 if tiles is None else int(tiles.shape[0])
    check(lib().et_tile_densify(_p(row_ptr), _p(row_off) if nnz else None,
                                _p(tiles) if nnz else None, c_int(nnz), c_int(inn), c_int(out),
                                _p(dense), _stream()), "et_tile_densify")
    # a weight must be complete before the first Linear call that uses it: those calls fetch
    # weights ahead of their predecessors on the stream
    torch.cuda.current_stream().synchronize()
    return dense


def linear_tile_packed(x, pk: "PackedTiles", bias=None, act=ACT_NONE):
    T, inn = x.shape
    y = _empty((T, pk.out), x)
    check(lib().et_linear_tile_packed_fwd(_p(pk.row_ptr), _p(pk.pk_mask), _p(pk.pk_off),
                                          _p(pk.tiles) if pk.nnz else None, c_int(pk.nnz),
                                          _p(bias), _p(x), _p(y), c_int(T), c_int(inn),
                                          c_int(pk.out), c_int(act), _stream()),
          "et_linear_tile_packed_fwd")
    return y


def linear_row(x, row_id, rows, out, bias=None, act=ACT_NONE):
    T, inn = x.shape
    y = _empty((T, out), x)
    nn = 0 if row_id is None else int(row_id.shape[0])
    check(lib().et_linear_row_fwd(_p(row_id) if nn else None, _p(rows) if nn else None, c_int(nn),
                                  _p(bias), _p(x), _p(y), c_int(T), c_int(inn), c_int(out),
                                  c_int(act), _stream()), "et_linear_row_fwd")
    return y


def linear_row_compressed(x, row_id, rows, bias=None):
    T, inn = x.shape
    nn = int(row_id.shape[0])
    y = _empty((T, nn), x)
    check(lib().et_linear_row_compressed_fwd(_p(row_id), _p(rows), c_int(nn), _p(bias), _p(x),
                                             _p(y), c_int(T), c_int(inn), _stream()),
          "et_linear_row_compressed_fwd")
    return y


def linear_col(x, col_id, cols, bias=None, act=ACT_NONE, scratch=None):
    T, inn = x.shape
    out, nn = cols.shape
    y = _empty((T, out), x)
    if scratch is None:
        scratch = _empty((T, nn), x)
    check(lib().et_linear_col_fwd(_p(col_id), _p(cols), c_int(nn), _p(bias), _p(x), _p(y),
                                  c_int(T), c_int(inn), c_int(out), c_int(act), _p(scratch),
                                  c_size_t(scratch.numel() * 2), _stream()), "et_linear_col_fwd")
    return y


def linear_col_noalloc(x, col_id, cols, y, bias=None, act=ACT_NONE):
    """Column-pruned Linear through the entry point that uses the library's built-in scratch;
    the caller supplies the output tensor too, so nothing is allocated here either."""
    T, inn = x.shape
    out, nn = cols.shape
    check(lib().et_linear_col_noalloc_fwd(_p(col_id), _p(cols), c_int(nn), _p(bias), _p(x), _p(y),
                                          c_int(T), c_int(inn), c_int(out), c_int(act),
                                          _stream()), "et_linear_col_noalloc_fwd")
    return y


def linear_1x16(x, tile_idx, row_idx, data, out, bias=None, act=ACT_NONE):
    T, inn = x.shape
    y = _empty((T, out), x)
    nvec = 0 if row_idx is None else int(row_idx.shape[0])
    check(lib().et_linear_1x16_fwd(_p(tile_idx), _p(row_idx) if nvec else None,
                                   _p(data) if nvec else None, c_int(nvec), _p(bias), _p(x), _p(y),
                                   c_int(T), c_int(inn), c_int(out), c_int(act), _stream()),
          "et_linear_1x16_fwd")
    return y


def v1x16_prefer_dense(inn: int, out: int, nvec: int) -> bool:
    """Plan-time choice for 1x16-vector weights: True when the dense GEMM on the expanded weight
    is expected to beat the vector kernel."""
    return bool(lib().et_1x16_prefer_dense(c_int(inn), c_int(out), c_int(nvec)))


def v1x16_densify(tile_idx, row_idx, data, inn: int, out: int):
    """dense[out, in] fp16 from device 1x16 arrays (pruned vectors zero)."""
    import torch
    dense = torch.empty((out, inn), dtype=torch.float16, device=tile_idx.device)
    nvec = 0 if row_idx is None else int(row_idx.shape[0])
    check(lib().et_1x16_densify(_p(tile_idx), _p(row_idx) if nvec else None,
                                _p(data) if nvec else None, c_int(nvec), c_int(inn), c_int(out),
                                _p(dense), _stream()), "et_1x16_densify")
    torch.cuda.current_stream().synchronize()  # weights must be complete before their first use
    return dense


def linear_csr(x, indptr, indices, data, out, bias=None, act=ACT_NONE):
    T, inn = x.shape
    y = _empty((T, out), x)
    nnz = 0 if indices is None else int(indices.shape[0])
    check(lib().et_linear_csr_fwd(_p(indptr), _p(indices) if nnz else None,
                                  _p(data) if nnz else None, c_int(nnz), _p(bias), _p(x), _p(y),
                                  c_int(T), c_int(inn), c_int(out), c_int(act), _stream()),
          "et_linear_csr_fwd")
    return y


# ---- normalisation / element-wise ---------------------------------------------------------

def skip_layernorm(src, skip, gamma, beta, out=None):
    rows, size = src.shape
    out = _empty((rows, size), src) if out is None else out
    check(lib().et_skip_layernorm_fwd(_p(src), _p(skip), _p(gamma), _p(beta), _p(out), c_int(rows),
                                      c_int(size), _stream()), "et_skip_layernorm_fwd")
    return out


def linear_skip_layernorm(x, w, bias, resid, gamma, beta, out=None):
    """LayerNorm(x w^T + bias + resid) * gamma + beta in one kernel (out: 256..1024, % 128)."""
    T, inn = x.shape
    n = w.shape[0]
    y = _empty((T, n), x) if out is None else out
    check(lib().et_linear_skip_layernorm_fwd(_p(x), _p(w), _p(bias), _p(resid), _p(gamma),
                                             _p(beta), _p(y), c_int(T), c_int(inn), c_int(n),
                                             _stream()), "et_linear_skip_layernorm_fwd")
    return y


def layernorm(src, gamma, beta):
    rows, size = src.shape
    out = _empty((rows, size), src)
    check(lib().et_layernorm_fwd(_p(src), _p(gamma), _p(beta), _p(out), c_int(rows), c_int(size),
                                 _stream()), "et_layernorm_fwd")
    return out


def act(x, kind, inplace=False):
    out = x if inplace else _empty(tuple(x.shape), x)
    check(lib().et_act_fwd(_p(x), _p(out), c_size_t(x.numel()), c_int(kind), _stream()),
          "et_act_fwd")
    return out


def bias_add_(data, bias):
    rows, cols = data.shape
    check(lib().et_bias_add_fwd(_p(data), _p(bias), c_int(rows), c_int(cols), _stream()),
          "et_bias_add_fwd")
    return data


# ---- attention ----------------------------------------------------------------------------

def attention(q, k, v, batch, seq, nhead, dh_qk, dh_v, mask_kind=MASK_NONE, mask=None,
              valid_len=None, scale=None, ldq=None, ldk=None, ldv=None, out=None):
    """q/k/v: fp16 tensors (possibly views into one fused buffer); ld* default to the row
    stride of each tensor; `out`: optional preallocated result."""
    ldq = q.stride(0) if ldq is None else ldq
    ldk = k.stride(0) if ldk is None else ldk
    ldv = v.stride(0) if ldv is None else ldv
    z = _empty((batch * seq, nhead * dh_v), q) if out is None else out
    scale = (1.0 / dh_qk ** 0.5) if scale is None else scale
    check(lib().et_attention_fwd(_p(q), _p(k), _p(v), _p(z), c_int(batch), c_int(seq),
                                 c_int(nhead), c_int(dh_qk), c_int(dh_v), c_int(ldq), c_int(ldk),
                                 c_int(ldv), c_int(nhead * dh_v), c_int(mask_kind), _p(mask),
                                 _p(valid_len), c_float(scale), _stream()), "et_attention_fwd")
    return z


def qkv_attention(x, wqkv, bqkv, batch, seq, nhead, kdim, vdim, mask_kind=MASK_NONE, mask=None,
                  valid_len=None, scale=None):
    """Fused Q/K/V projection + attention (seq <= 128, 64-wide heads)."""
    z = _empty((batch * seq, vdim), x)
    scale = (1.0 / (kdim // nhead) ** 0.5) if scale is None else scale
    check(lib().et_qkv_attention_fwd(_p(x), _p(wqkv), _p(bqkv), _p(z), c_int(batch), c_int(seq),
                                     c_int(x.shape[1]), c_int(nhead), c_int(kdim), c_int(vdim),
                                     c_int(mask_kind), _p(mask), _p(valid_len), c_float(scale),
                                     _stream()), "et_qkv_attention_fwd")
    return z


def attention_pruned_v(q, k, vc, col_id, head_ptr, batch, seq, nhead, dh_qk, dh_v,
                       mask_kind=MASK_NONE, mask=None, valid_len=None, scale=None):
    z = _empty((batch * seq, nhead * dh_v), q)
    scale = (1.0 / dh_qk ** 0.5) if scale is None else scale
    check(lib().et_attention_pruned_v_fwd(_p(q), _p(k), _p(vc), _p(col_id), _p(head_ptr),
                                          c_int(int(col_id.shape[0])), _p(z), c_int(batch),
                                          c_int(seq), c_int(nhead), c_int(dh_qk), c_int(dh_v),
                                          c_int(q.stride(0)), c_int(k.stride(0)),
                                          c_int(nhead * dh_v), c_int(mask_kind), _p(mask),
                                          _p(valid_len), c_float(scale), _stream()),
          "et_attention_pruned_v_fwd")
    return z


def attention_fuse_o(q, k, v, o_row_ptr, o_row_off, o_tiles, o_bias, batch, seq, nhead, dh_qk,
                     dh_v, emdim, mask_kind=MASK_NONE, mask=None, valid_len=None, scale=None,
                     single_launch=False):
    """Attention + tile-CSR output projection (Attention/kernel_fuseO.cu:254-290);
    single_launch=True runs both in one kernel."""
    z = _empty((batch * seq, nhead * dh_v), q)
    out = _empty((batch * seq, emdim), q)
    scale = (1.0 / dh_qk ** 0.5) if scale is None else scale
    fn = lib().et_attention_fuse_o_single_launch_fwd if single_launch else lib().et_attention_fuse_o_fwd
    check(fn(_p(q), _p(k), _p(v), _p(mask), _p(z), _p(o_row_ptr),
                                        _p(o_row_off), _p(o_tiles), c_int(int(o_tiles.shape[0])),
                                        _p(o_bias), _p(out), c_int(batch), c_int(seq),
                                        c_int(nhead), c_int(dh_qk), c_int(dh_v),
                                        c_int(q.stride(0)), c_int(k.stride(0)),
                                        c_int(v.stride(0)), c_int(emdim), c_int(mask_kind),
                                        _p(valid_len), c_float(scale), _stream()),
          "et_attention_fuse_o_fwd")
    return out


def linear_vo(x, w_vo, bias, batch, seq, nhead, emdim):
    vo = _empty((batch * nhead * seq, emdim), x)
    check(lib().et_linear_vo_fwd(_p(x), _p(w_vo), _p(bias), _p(vo), c_int(batch), c_int(seq),
                                 c_int(nhead), c_int(emdim), _stream()), "et_linear_vo_fwd")
    return vo


def fused_vo_attention(q, k, vo, bias_o, batch, seq, nhead, dh_qk, emdim, mask_kind=MASK_NONE,
                       mask=None, valid_len=None, scale=None):
    out = _empty((batch * seq, emdim), q)
    scale = (1.0 / dh_qk ** 0.5) if scale is None else scale
    check(lib().et_fused_vo_attention_fwd(_p(q), _p(k), _p(vo), _p(bias_o), _p(out), c_int(batch),
                                          c_int(seq), c_int(nhead), c_int(dh_qk), c_int(emdim),
                                          c_int(q.stride(0)), c_int(k.stride(0)),
                                          c_int(mask_kind), _p(mask), _p(valid_len),
                                          c_float(scale), _stream()),
          "et_fused_vo_attention_fwd")
    return out


# ---- encoder layer / stack ----------------------------------------------------------------

def linear_vo_pruned(x, w_vo_c, bias, batch, seq, nhead, emdim):
    """w_vo_c: [nhead, emdim, nnz_col]; returns VOc [batch * nhead * seq, nnz_col]."""
    nnz = int(w_vo_c.shape[2])
    vo = _empty((batch * nhead * seq, nnz), x)
    check(lib().et_linear_vo_pruned_fwd(_p(x), _p(w_vo_c), _p(bias), _p(vo), c_int(batch), c_int(seq),
                                        c_int(nhead), c_int(emdim), c_int(nnz), _stream()),
          "et_linear_vo_pruned_fwd")
    return vo


def fused_vo_attention_pruned(q, k, vo_c, col_id, bias_o, batch, seq, nhead, dh_qk, emdim,
                              mask_kind=MASK_NONE, mask=None, valid_len=None, scale=None):
    nnz = int(vo_c.shape[1])
    scratch = _empty((batch * seq, nnz), q)
    out = _empty((batch * seq, emdim), q)
    scale = (1.0 / dh_qk ** 0.5) if scale is None else scale
    check(lib().et_fused_vo_attention_pruned_fwd(
        _p(q), _p(k), _p(vo_c), _p(col_id), c_int(nnz), _p(bias_o), _p(scratch), _p(out),
        c_int(batch), c_int(seq), c_int(nhead), c_int(dh_qk), c_int(emdim), c_int(q.stride(0)),
        c_int(k.stride(0)), c_int(mask_kind), _p(mask), _p(valid_len), c_float(scale), _stream()),
        "et_fused_vo_attention_pruned_fwd")
    return out


class EncoderLayer:
    """Device-resident weights of one encoder layer plus the et_encoder_layer_t that
    describes them.  `weights` is the dict of numpy fp16 arrays synth.encoder_layer_weights
    returns; tile_sparse=True stores the four Linear layers in re-packed tile-CSR form,
    tile_sparse="unpacked" in the reference's tile-CSR order, and tile_sparse="auto" lets
    et_tile_prefer_dense choose per weight between the packed tile kernel and the dense GEMM
    on the expanded weight.

    `formats` overrides that per weight ("wqkv", "wo", "w1", "w2"): "dense", "1x16" (the vector
    kernel), "1x16_auto" (et_1x16_prefer_dense chooses between it and the dense GEMM on the
    expanded weight), "csr", ("row", ids) (kept output rows) or ("col", ids) (kept input
    columns).  ("row", ids) on "w1" with ("col", ids) on "w2" over the same `ids` array object
    describes pruned hidden units of the feed-forward block: both products run at the kept
    width."""

    def __init__(self, weights: dict, nhead: int, act_kind: int = ACT_GELU, device="cuda",
                 tile_sparse: bool = False, formats: dict | None = None):
        import numpy as np
        import torch
        self._keep = []
        formats = formats or {}
        id_cache = {}  # id(list object) -> device tensor, so that equal lists share one array

        def dev(a):
            t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
            self._keep.append(t)
            return t

        def dev_ids(ids):
            if id(ids) not in id_cache:
                id_cache[id(ids)] = dev(np.ascontiguousarray(ids, dtype=np.int32))
            return id_cache[id(ids)]

        def lin(wname, bname):
            W = weights[wname]
            d = LinearDesc()
            d.out, d.in_ = int(W.shape[0]), int(W.shape[1])
            d.bias = weights[bname] is not None and dev(weights[bname]).data_ptr() or None
            fmt = formats.get(wname)
            if fmt is not None and fmt != "dense":
                kind = fmt if isinstance(fmt, str) else fmt[0]
                if kind in ("1x16", "1x16_auto"):
                    tidx, ridx, data = synth.dense_to_1x16(W)
                    nvec = int(ridx.shape[0])
                    dt, dr = dev(tidx), dev(ridx) if nvec else None
                    dd = dev(data) if nvec else None
                    if kind == "1x16_auto" and v1x16_prefer_dense(d.in_, d.out, nvec):
                        dense = v1x16_densify(dt, dr, dd, d.in_, d.out)
                        self._keep.append(dense)
                        d.format, d.weight = FMT_DENSE, dense.data_ptr()
                    else:
                        d.format, d.nnz_tiles = FMT_1X16, nvec
                        d.row_ptr = dt.data_ptr()
                        if nvec:
                            d.row_off, d.weight = dr.data_ptr(), dd.data_ptr()
                elif kind == "row":
                    ids = fmt[1]
                    _, rows = synth.dense_to_row(W, np.asarray(ids))
                    d.format, d.nnz_tiles = FMT_ROW, int(len(ids))
                    d.row_ptr, d.weight = dev_ids(ids).data_ptr(), dev(rows).data_ptr()
                elif kind == "col":
                    ids = fmt[1]
                    _, cols = synth.dense_to_col(W, np.asarray(ids))
                    d.format, d.nnz_tiles = FMT_COL, int(len(ids))
                    d.row_ptr, d.weight = dev_ids(ids).data_ptr(), dev(cols).data_ptr()
                elif kind == "csr":
                    indptr, indices, data = synth.dense_to_csr(W)
                    d.format, d.nnz_tiles = FMT_CSR, int(indices.shape[0])
                    d.row_ptr = dev(indptr).data_ptr()
                    if d.nnz_tiles:
                        d.row_off, d.weight = dev(indices).data_ptr(), dev(data).data_ptr()
                else:
                    raise EtError(f"unknown weight format {fmt!r}")
            elif tile_sparse and fmt is None:
                rp, ro, tiles = synth.dense_to_tile(W)
                d.nnz_tiles = int(tiles.shape[0])
                # the fused projection + attention kernel needs a dense Q/K/V weight and beats
                # the tile kernel followed by the attention kernel at any sparsity below ~97 %
                fusable = wname == "wqkv" and d.out % (3 * 64) == 0 and d.out // 3 == 64 * nhead
                if tile_sparse == "auto" and (fusable or
                                              tile_prefer_dense(d.in_, d.out, d.nnz_tiles)):
                    dense = tile_densify(dev(rp), dev(ro) if d.nnz_tiles else None,
                                         dev(tiles) if d.nnz_tiles else None, d.in_, d.out)
                    self._keep.append(dense)
                    d.format = FMT_DENSE
                    d.nnz_tiles = 0
                    d.weight = dense.data_ptr()
                elif tile_sparse == "unpacked":
                    d.format = FMT_TILE
                    d.row_ptr = dev(rp).data_ptr()
                    if d.nnz_tiles:
                        d.row_off = dev(ro).data_ptr()
                        d.weight = dev(tiles).data_ptr()
                else:
                    pk = PackedTiles(rp, ro, tiles, d.in_, d.out, device)
                    self._keep.append(pk)
                    d.format = FMT_TILE_PACKED
                    d.row_ptr = pk.row_ptr.data_ptr()
                    d.pk_mask = pk.pk_mask.data_ptr()
                    d.pk_off = pk.pk_off.data_ptr()
                    if d.nnz_tiles:
                        d.weight = pk.tiles.data_ptr()
            else:
                d.format = FMT_DENSE
                d.weight = dev(W).data_ptr()
            return d

        self.desc = EncoderLayerDesc()
        self.desc.qkv = lin("wqkv", "bqkv")
        self.desc.o = lin("wo", "bo")
        self.desc.ffn1 = lin("w1", "b1")
        self.desc.ffn2 = lin("w2", "b2")
        self.desc.ln1_gamma = dev(weights["ln1_g"]).data_ptr()
        self.desc.ln1_beta = dev(weights["ln1_b"]).data_ptr()
        self.desc.ln2_gamma = dev(weights["ln2_g"]).data_ptr()
        self.desc.ln2_beta = dev(weights["ln2_b"]).data_ptr()
        hidden = int(weights["wo"].shape[0])
        vdim = int(weights["wo"].shape[1])
        kdim = (int(weights["wqkv"].shape[0]) - vdim) // 2
        self.desc.hidden, self.desc.nhead = hidden, nhead
        self.desc.kdim, self.desc.vdim = kdim, vdim
        self.desc.ff = int(weights["w1"].shape[0])
        self.desc.act = act_kind
        self.hidden = hidden

    def workspace_bytes(self, batch: int, seq: int) -> int:
        return int(lib().et_encoder_layer_workspace_bytes(ctypes.byref(self.desc), c_int(batch),
                                                          c_int(seq)))

    def forward(self, x, out, batch, seq, workspace, mask_kind=MASK_NONE, mask=None,
                valid_len=None):
        check(lib().et_encoder_layer_fwd(ctypes.byref(self.desc), _p(x), _p(out), c_int(batch),
                                         c_int(seq), c_int(mask_kind), _p(mask), _p(valid_len),
                                         _p(workspace), c_size_t(workspace.numel() *
                                                                 workspace.element_size()),
                                         _stream()), "et_encoder_layer_fwd")
        return out


class HeadParallelLayer:
    """One encoder layer over `job.world` GPUs for a batch that cannot be sharded (one long
    sequence).  The attention block is cut into (head, query range) work units dealt out evenly
    (sharding.head_parallel_plan); every rank projects Q, K, V for the heads its units touch,
    attends over its units and multiplies by those heads' columns of the output projection
    (et_encoder_attention_units_fwd); ONE all-reduce adds the partial [T, hidden] sums; the
    LayerNorms and the FFN run replicated on the full layer (et_encoder_after_attention_fwd,
    the same fused kernels as et_encoder_layer_fwd).  `weights` is the full layer (numpy fp16).
    reduce_dtype "fp16" sums fp16 partials (6 MB per 4096 x 768 layer), "fp32" fp32 partials."""

    def __init__(self, weights: dict, nhead: int, job, act_kind: int = ACT_GELU, device="cuda",
                 reduce_dtype: str = "fp16"):
        import numpy as np
        import torch
        if reduce_dtype not in ("fp16", "fp32"):
            raise EtError("reduce_dtype must be 'fp16' or 'fp32'")
        self.job, self.nhead, self.f32 = job, nhead, reduce_dtype == "fp32"
        self.device = device
        self.full = EncoderLayer(weights, nhead, act_kind, device=device)
        self.weights = weights
        self._plans = {}  # seq -> (local layer description, unit arrays, ...)
        self._keep = []
        self.hidden = self.full.hidden
        self.units_per_rank = None

    @staticmethod
    def units_of(nhead: int, world: int, rank: int, seq: int):
        return sharding.units_of_rank(nhead, world, rank, seq)

    def _plan(self, seq: int):
        import numpy as np
        import torch
        if seq in self._plans:
            return self._plans[seq]
        world, rank = self.job.world, self.job.rank
        _, per_rank, bpu = sharding.head_parallel_plan(self.nhead, world, seq)
        units = sharding.units_of_rank(self.nhead, world, rank, seq)
        heads = sorted({h for h, _ in units})
        sl = sharding.head_rows(self.weights, self.nhead, heads)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        wqkv, bqkv, wo = dev(sl["wqkv"]), dev(sl["bqkv"]), dev(sl["wo"])
        bo = dev(self.weights["bo"]) if (rank == 0 and not self.f32) else None
        self._keep += [wqkv, bqkv, wo, bo]
        d = EncoderLayerDesc()
        ctypes.memmove(ctypes.byref(d), ctypes.byref(self.full.desc), ctypes.sizeof(d))
        nh = len(heads)
        d.nhead, d.kdim, d.vdim = nh, nh * sl["dh_qk"], nh * sl["dh_v"]
        d.qkv.format, d.qkv.in_, d.qkv.out = FMT_DENSE, self.hidden, int(wqkv.shape[0])
        d.qkv.weight, d.qkv.bias = wqkv.data_ptr(), bqkv.data_ptr()
        d.o.format, d.o.in_, d.o.out = FMT_DENSE, int(wo.shape[1]), self.hidden
        d.o.weight, d.o.bias = wo.data_ptr(), (bo.data_ptr() if bo is not None else None)
        uh = (ctypes.c_int32 * len(units))(*[heads.index(h) for h, _ in units])
        uf = (ctypes.c_int32 * len(units))(*[f for _, f in units])
        self.units_per_rank = per_rank
        plan = (d, uh, uf, len(units), bpu)
        self._plans[seq] = plan
        return plan

    def _workspace(self, d, batch, seq, like):
        import torch
        ws_bytes = max(int(lib().et_encoder_layer_workspace_bytes(ctypes.byref(d), c_int(batch),
                                                                  c_int(seq))),
                       self.full.workspace_bytes(batch, seq))
        if getattr(self, "_ws", None) is None or self._ws.numel() < ws_bytes:
            self._ws = torch.empty(ws_bytes, dtype=torch.uint8, device=like.device)
        return self._ws

    def partial_sum(self, x, batch: int, seq: int, mask_kind=MASK_NONE, mask=None, valid_len=None,
                    out_ptr: int | None = None):
        """This rank's share of the attention block: [T, hidden] (fp16 or fp32), as a new tensor
        or written at the device address `out_ptr` (then nothing is returned)."""
        import torch
        d, uh, uf, n_units, bpu = self._plan(seq)
        ws = self._workspace(d, batch, seq, x)
        partial = None
        if out_ptr is None:
            partial = torch.empty((batch * seq, self.hidden),
                                  dtype=torch.float32 if self.f32 else torch.float16, device=x.device)
        check(lib().et_encoder_attention_units_fwd(
            ctypes.byref(d), _p(x), _p(partial) if out_ptr is None else c_void_p(out_ptr),
            c_int(1 if self.f32 else 0), c_int(batch), c_int(seq),
            c_int(mask_kind), _p(mask), _p(valid_len), uh, uf, c_int(n_units), c_int(bpu),
            _p(ws), c_size_t(ws.numel()), _stream()), "et_encoder_attention_units_fwd")
        return partial

    def finish(self, attn_sum, x, batch: int, seq: int):
        """The replicated rest of the layer on the summed attention block."""
        d = self._plan(seq)[0]
        ws = self._workspace(d, batch, seq, x)
        out = _empty((batch * seq, self.hidden), x)
        check(lib().et_encoder_after_attention_fwd(
            ctypes.byref(self.full.desc), _p(attn_sum), c_int(1 if self.f32 else 0), _p(x), _p(out),
            c_int(batch), c_int(seq), _p(ws), c_size_t(ws.numel()), _stream()),
            "et_encoder_after_attention_fwd")
        return out

    def forward(self, x, batch: int, seq: int, mask_kind=MASK_NONE, mask=None, valid_len=None,
                skip_allreduce: bool = False):
        """skip_allreduce=True leaves out the exchange step (timing aid: the result is then the
        layer applied to this rank's partial sum only)."""
        partial = self.partial_sum(x, batch, seq, mask_kind, mask, valid_len)
        if self.job.world > 1 and not skip_allreduce:
            import torch.distributed as dist
            dist.all_reduce(partial)  # the layer's one exchange step
        return self.finish(partial, x, batch, seq)

    # ---- the same layer with the exchange done by this library's kernels over peer memory ----
    def ffn(self, y_ptr: int, x, batch: int, seq: int):
        d = self._plan(seq)[0]
        ws = self._workspace(d, batch, seq, x)
        out = _empty((batch * seq, self.hidden), x)
        check(lib().et_encoder_ffn_fwd(ctypes.byref(self.full.desc), c_void_p(y_ptr), _p(out), c_int(batch),
                                       c_int(seq), _p(ws), c_size_t(ws.numel()), _stream()),
              "et_encoder_ffn_fwd")
        return out

    def forward_peer(self, x, batch: int, seq: int, exchange: "PeerExchange", mask_kind=MASK_NONE,
                     mask=None, valid_len=None):
        """forward() with the partial sums pulled by their owner ranks through peer mappings,
        summed, normalised and gathered by peer stores (PeerExchange) instead of a library
        all-reduce.  fp16 partials."""
        if self.f32:
            raise EtError("the peer exchange sums fp16 partials")
        self.partial_sum(x, batch, seq, mask_kind, mask, valid_len, out_ptr=exchange.partial())
        exchange.epoch += 1
        d = self.full.desc  # (the output projection's bias is inside rank 0's partial)
        exchange.reduce_layernorm(x, None, c_void_p(d.ln1_gamma), c_void_p(d.ln1_beta), publish_ready=True)
        exchange.wait()
        return self.ffn(exchange.y(), x, batch, seq)

    def forward_peer_sharded(self, x, batch: int, seq: int, exchange: "PeerExchange", mask_kind=MASK_NONE,
                             mask=None, valid_len=None, phase: str = "all"):
        """forward_peer() with the feed-forward block and the second LayerNorm run on THIS RANK'S
        token rows only (they act on tokens independently) and the finished rows passed to every
        rank: a reduce-scatter after the output projection and an all-gather after the layer, the
        bytes of one all-reduce.  Returns the layer output as a view of the exchange buffer's
        out[slot] (valid until the layer call after next).  batch must be 1.
        phase (single-GPU emulation of several ranks): "partial" / "reduce" / "ffn" / "wait" run
        one step each so that every rank's step can run before the next step of any rank."""
        if self.f32:
            raise EtError("the peer exchange sums fp16 partials")
        if batch != 1:
            raise EtError("the token-sharded form handles one sequence")
        T = seq
        if phase in ("all", "partial"):
            self.partial_sum(x, batch, seq, mask_kind, mask, valid_len, out_ptr=exchange.partial())
            exchange.epoch += 1
            if phase == "partial":
                exchange.signal()
        d = self.full.desc
        if phase in ("all", "reduce"):
            exchange.reduce_layernorm(x, None, c_void_p(d.ln1_gamma), c_void_p(d.ln1_beta),
                                      publish_ready=(phase == "all"), gather=False)
        slot = exchange.epoch & 1
        first, n = exchange.rows()
        if phase in ("all", "ffn"):
            if n > 0:
                dl = self._plan(seq)[0]
                ws = self._workspace(dl, batch, seq, x)
                yp = exchange.y() + first * self.hidden * 2
                op = exchange.out(slot) + first * self.hidden * 2
                check(lib().et_encoder_ffn_fwd(ctypes.byref(self.full.desc), c_void_p(yp), c_void_p(op),
                                               c_int(1), c_int(n), _p(ws), c_size_t(ws.numel()), _stream()),
                      "et_encoder_ffn_fwd")
            exchange.allgather_rows(slot)
        if phase in ("all", "wait"):
            exchange.wait()
        return device_view(exchange.out(slot), (T, self.hidden), x.device)


class _DeviceArray:
    """A raw device address as a zero-copy torch tensor (torch.as_tensor on this object)."""

    def __init__(self, ptr: int, shape, typestr: str = "<f2"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


def device_view(ptr: int, shape, device):
    import torch
    return torch.as_tensor(_DeviceArray(ptr, shape), device=device)


class PeerExchange:
    """The ranks' exchange buffers for the head-parallel layer over peer memory: one buffer per
    rank (et_peer_buffer_create), every other rank's buffer mapped through its CUDA IPC handle.
    `handles` may be given by the caller; with a torch.distributed job they are all-gathered.
    For a single-process emulation of several ranks on one GPU use PeerExchange.local()."""

    def __init__(self, job, T: int, hidden: int):
        """Collective over the job's ranks.  Every rank takes part in both collective steps (the
        all-gather of the handles, the agreement on success) whatever happens locally, so that a
        failure on one rank (no peer access, IPC refused) raises EtError on ALL ranks instead of
        leaving the others waiting."""
        import torch
        import torch.distributed as dist
        self.world, self.rank, self.T, self.hidden = job.world, job.rank, T, hidden
        self.epoch = 0
        self.own, self._opened = None, []
        failure = None
        handle = (ctypes.c_ubyte * 64)()
        try:
            nbytes = ctypes.c_size_t(0)
            check(lib().et_peer_buffer_bytes(c_int(self.world), c_int(T), c_int(hidden), ctypes.byref(nbytes)),
                  "et_peer_buffer_bytes")
            own = c_void_p(None)
            check(lib().et_peer_buffer_create(nbytes, ctypes.byref(own), handle), "et_peer_buffer_create")
            self.own = own.value
        except Exception as e:  # noqa: BLE001 - reported after the collective steps
            failure = e
        ptrs = [None] * self.world
        ptrs[self.rank] = self.own
        if self.world > 1:
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=job.device)
            every = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(every, mine)
            if failure is None:
                try:
                    for r in range(self.world):
                        if r == self.rank:
                            continue
                        h = (ctypes.c_ubyte * 64)(*every[r].cpu().tolist())
                        p = c_void_p(None)
                        check(lib().et_peer_buffer_open(h, ctypes.byref(p)), "et_peer_buffer_open")
                        ptrs[r] = p.value
                        self._opened.append(p.value)
                except Exception as e:  # noqa: BLE001
                    failure = e
            ok = torch.tensor([0 if failure is not None else 1], dtype=torch.int32, device=job.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                self.close()
                raise EtError(f"peer exchange unavailable on at least one rank (this rank: {failure!r})")
        elif failure is not None:
            raise EtError(f"peer exchange unavailable: {failure!r}")
        self.ptrs = (c_void_p * self.world)(*ptrs)

    @classmethod
    def local(cls, world: int, T: int, hidden: int):
        """`world` exchange objects in ONE process whose buffers all live on the current GPU
        (tests: the ranks' kernels then run one after the other, phase by phase)."""
        nbytes = ctypes.c_size_t(0)
        check(lib().et_peer_buffer_bytes(c_int(world), c_int(T), c_int(hidden), ctypes.byref(nbytes)),
              "et_peer_buffer_bytes")
        bufs = []
        for _ in range(world):
            own, handle = c_void_p(None), (ctypes.c_ubyte * 64)()
            check(lib().et_peer_buffer_create(nbytes, ctypes.byref(own), handle), "et_peer_buffer_create")
            bufs.append(own.value)
        out = []
        for r in range(world):
            ex = cls.__new__(cls)
            ex.world, ex.rank, ex.T, ex.hidden, ex.epoch = world, r, T, hidden, 0
            ex.own, ex._opened = bufs[r], []
            ex.ptrs = (c_void_p * world)(*bufs)
            out.append(ex)
        return out

    def y(self):
        """This rank's copy of the LN1 output [T, hidden] as a torch view of the buffer."""
        import torch
        yp = c_void_p(None)
        check(lib().et_peer_buffer_y(c_void_p(self.own), c_int(self.world), c_int(self.T), c_int(self.hidden),
                                     ctypes.byref(yp)), "et_peer_buffer_y")
        return yp.value

    def partial(self):
        """Device address of this rank's partial [T, hidden] fp16 inside its exchange buffer."""
        return self.own

    def signal(self):
        check(lib().et_hp_signal_partial_fwd(self.ptrs, c_int(self.rank), c_int(self.world), c_int(self.T),
                                             c_int(self.hidden), c_int(self.epoch), _stream()),
              "et_hp_signal_partial_fwd")

    def reduce_layernorm(self, x, bias, gamma, beta, publish_ready: bool = False, gather: bool = True):
        """bias / gamma / beta: device tensors or raw device addresses (c_void_p).
        publish_ready: also do signal()'s job (one rank per GPU only).  gather=False keeps y
        local (token-sharded form: only this rank's rows are computed and valid)."""
        vp = lambda a: a if isinstance(a, c_void_p) else _p(a)
        check(lib().et_hp_reduce_layernorm_fwd(self.ptrs, _p(x), vp(bias), vp(gamma), vp(beta),
                                               c_int(self.rank), c_int(self.world), c_int(self.T),
                                               c_int(self.hidden), c_int(self.epoch),
                                               c_int(1 if publish_ready else 0), c_int(1 if gather else 0),
                                               _stream()),
              "et_hp_reduce_layernorm_fwd")

    def rows(self):
        """(first row, number of rows) this rank owns."""
        per = (self.T + self.world - 1) // self.world
        first = self.rank * per
        return first, max(0, min(per, self.T - first))

    def out(self, slot: int):
        """Device address of out[slot] [T, hidden] fp16 in this rank's buffer."""
        op = c_void_p(None)
        check(lib().et_peer_buffer_out(c_void_p(self.own), c_int(self.world), c_int(self.T), c_int(self.hidden),
                                       c_int(slot), ctypes.byref(op)), "et_peer_buffer_out")
        return op.value

    def allgather_rows(self, slot: int):
        check(lib().et_hp_allgather_rows_fwd(self.ptrs, c_int(self.rank), c_int(self.world), c_int(self.T),
                                             c_int(self.hidden), c_int(self.epoch), c_int(slot), _stream()),
              "et_hp_allgather_rows_fwd")

    def wait(self):
        check(lib().et_hp_wait_fwd(c_void_p(self.own), c_int(self.world), c_int(self.T), c_int(self.hidden),
                                   c_int(self.epoch), _stream()), "et_hp_wait_fwd")

    def close(self):
        for p in self._opened:
            lib().et_peer_buffer_close(c_void_p(p))
        self._opened = []
        if self.own:
            lib().et_peer_buffer_destroy(c_void_p(self.own))
            self.own = None


class EncoderStack:
    """N chained encoder layers.  The batch can be cut into `lanes` groups of sequences that
    run through the whole stack on streams of their own (sequences are independent), so that
    the kernels of one group fill the SMs another group's kernels leave idle; each group has
    its own workspace, all share two ping-pong activation buffers."""

    def __init__(self, layers, batch: int, seq: int, device="cuda", lanes: int = 1):
        import torch
        self.layers = list(layers)
        self.batch, self.seq = batch, seq
        lanes = max(1, min(lanes, batch))
        base, extra = divmod(batch, lanes)
        self.groups = []  # (first sequence, number of sequences)
        first = 0
        for i in range(lanes):
            n = base + (1 if i < extra else 0)
            self.groups.append((first, n))
            first += n
        hidden = self.layers[0].hidden
        self.workspaces = []
        for _, n in self.groups:
            ws = max(l.workspace_bytes(n, seq) for l in self.layers)
            if ws == 0:
                raise EtError("invalid encoder layer description")
            self.workspaces.append(torch.empty(ws, dtype=torch.uint8, device=device))
        self.workspace = self.workspaces[0]
        self.buf = [torch.empty((batch * seq, hidden), dtype=torch.float16, device=device)
                    for _ in range(2)]
        self.streams = [torch.cuda.Stream(device=device) for _ in self.groups[1:]]
        self.events = [(torch.cuda.Event(), torch.cuda.Event()) for _ in self.groups[1:]]

    def _run_group(self, g, x, mask_kind, mask, valid_len):
        first, n = self.groups[g]
        r0, r1 = first * self.seq, (first + n) * self.seq
        cur = x[r0:r1]
        vl = None if valid_len is None else valid_len[first:first + n]
        for i, layer in enumerate(self.layers):
            out = self.buf[i & 1][r0:r1]
            layer.forward(cur, out, n, self.seq, self.workspaces[g], mask_kind, mask, vl)
            cur = out

    def forward(self, x, mask_kind=MASK_NONE, mask=None, valid_len=None):
        import torch
        main = torch.cuda.current_stream()
        for g in range(1, len(self.groups)):
            start, _ = self.events[g - 1]
            start.record(main)
            self.streams[g - 1].wait_event(start)
            with torch.cuda.stream(self.streams[g - 1]):
                self._run_group(g, x, mask_kind, mask, valid_len)
        self._run_group(0, x, mask_kind, mask, valid_len)
        for g in range(1, len(self.groups)):
            _, done = self.events[g - 1]
            done.record(self.streams[g - 1])
            main.wait_event(done)
        return self.buf[(len(self.layers) - 1) & 1]


class HostPipeline:
    """Serving loop over an EncoderStack for callers whose batches live in (pinned) host memory:
    `submit(x_host, y_host)` queues host-to-device copy, the stack (replayed from a CUDA graph)
    and device-to-host copy of one batch on three streams; with `depth` >= 2 input / output
    slots the copies of neighbouring batches overlap the compute of the current one.  `drain()`
    waits for everything queued.  Results land in the caller's `y_host` of each submit."""

    def __init__(self, stack: "EncoderStack", depth: int = 2, mask_kind=MASK_NONE, mask=None,
                 valid_len=None, use_graph: bool = True):
        import torch
        dev = stack.buf[0].device
        self.stack, self.depth = stack, max(1, depth)
        shape = tuple(stack.buf[0].shape)
        self.x_dev = [torch.empty(shape, dtype=torch.float16, device=dev) for _ in range(self.depth)]
        self.y_dev = [torch.empty(shape, dtype=torch.float16, device=dev) for _ in range(self.depth)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        mk = lambda: [torch.cuda.Event() for _ in range(self.depth)]
        self.ev_in, self.ev_run, self.ev_out = mk(), mk(), mk()
        self.count = 0
        self.kernels_per_step = 0
        self.graphs = []

        def run(slot):
            out = stack.forward(self.x_dev[slot], mask_kind, mask, valid_len)
            self.y_dev[slot].copy_(out)  # frees the stack's own buffer for the next batch

        with torch.cuda.stream(self.s_run):
            for slot in range(self.depth):
                run(slot)  # warm: sets kernel attributes before capture
            self.s_run.synchronize()
            for slot in range(self.depth):
                if use_graph:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.s_run):
                        run(slot)
                    self.graphs.append(g.replay)
                else:
                    self.graphs.append(lambda slot=slot: run(slot))
        torch.cuda.synchronize(dev)

    def submit(self, x_host, y_host) -> None:
        import torch
        slot = self.count % self.depth
        reuse = self.count >= self.depth
        with torch.cuda.stream(self.s_in):
            if reuse:
                self.s_in.wait_event(self.ev_run[slot])   # the stack has consumed this input slot
            self.x_dev[slot].copy_(x_host, non_blocking=True)
            self.ev_in[slot].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[slot])
            if reuse:
                self.s_run.wait_event(self.ev_out[slot])  # its previous result has left the device
            self.graphs[slot]()
            self.ev_run[slot].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[slot])
            y_host.copy_(self.y_dev[slot], non_blocking=True)
            self.ev_out[slot].record(self.s_out)
        self.count += 1

    def drain(self) -> None:
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()

