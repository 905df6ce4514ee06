"""numpy front end of the CPU oracle (oracle/et_oracle.cpp).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this
module; the product never does.  All functions take and return float32 numpy arrays
(fp16 inputs are widened first) and int32 index arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_float, c_int, c_long, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libet_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "et_oracle.cpp")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libet_oracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.orc_num_threads.restype = c_int
        for name in ("orc_dense_to_tile", "orc_dense_to_1x16", "orc_dense_to_csr"):
            getattr(_lib, name).restype = c_int
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Number of OpenMP threads of the following calls (overrides OMP_NUM_THREADS)."""
    lib().orc_set_num_threads(c_int(int(n)))


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def round_fp16(a):
    return _f(a).astype(np.float16).astype(np.float32)


def linear_dense(x, w, b=None, act=0):
    x, w = _f(x), _f(w)
    b = None if b is None else _f(b)
    T, inn = x.shape
    out = w.shape[0]
    y = np.empty((T, out), np.float32)
    lib().orc_linear_dense(_p(x), _p(w), _p(b), _p(y), c_int(T), c_int(inn), c_int(out), c_int(act))
    return y


def linear_tile(x, row_ptr, row_off, tiles, out, b=None, act=0):
    x, tiles = _f(x), _f(tiles)
    row_ptr, row_off = _i(row_ptr), _i(row_off)
    b = None if b is None else _f(b)
    T, inn = x.shape
    y = np.empty((T, out), np.float32)
    lib().orc_linear_tile(_p(row_ptr), _p(row_off), _p(tiles), _p(b), _p(x), _p(y), c_int(T),
                          c_int(inn), c_int(out), c_int(act))
    return y


def linear_row(x, row_id, rows, out, b=None, act=0):
    x, rows, row_id = _f(x), _f(rows), _i(row_id)
    b = None if b is None else _f(b)
    T, inn = x.shape
    y = np.empty((T, out), np.float32)
    lib().orc_linear_row(_p(row_id), _p(rows), c_int(len(row_id)), _p(b), _p(x), _p(y), c_int(T),
                         c_int(inn), c_int(out), c_int(act))
    return y


def linear_row_compressed(x, row_id, rows, b=None):
    x, rows, row_id = _f(x), _f(rows), _i(row_id)
    b = None if b is None else _f(b)
    T, inn = x.shape
    y = np.empty((T, len(row_id)), np.float32)
    lib().orc_linear_row_compressed(_p(row_id), _p(rows), c_int(len(row_id)), _p(b), _p(x), _p(y),
                                    c_int(T), c_int(inn))
    return y


def linear_col(x, col_id, cols, b=None, act=0):
    x, cols, col_id = _f(x), _f(cols), _i(col_id)
    b = None if b is None else _f(b)
    T, inn = x.shape
    out = cols.shape[0]
    y = np.empty((T, out), np.float32)
    lib().orc_linear_col(_p(col_id), _p(cols), c_int(len(col_id)), _p(b), _p(x), _p(y), c_int(T),
                         c_int(inn), c_int(out), c_int(act))
    return y


def linear_1x16(x, tile_idx, row_idx, data, out, b=None, act=0):
    x, data = _f(x), _f(data)
    tile_idx, row_idx = _i(tile_idx), _i(row_idx)
    b = None if b is None else _f(b)
    T, inn = x.shape
    y = np.empty((T, out), np.float32)
    lib().orc_linear_1x16(_p(tile_idx), _p(row_idx), _p(data), _p(b), _p(x), _p(y), c_int(T),
                          c_int(inn), c_int(out), c_int(act))
    return y


def linear_csr(x, indptr, indices, data, out, b=None, act=0):
    x, data = _f(x), _f(data)
    indptr, indices = _i(indptr), _i(indices)
    b = None if b is None else _f(b)
    T, inn = x.shape
    y = np.empty((T, out), np.float32)
    lib().orc_linear_csr(_p(indptr), _p(indices), _p(data), _p(b), _p(x), _p(y), c_int(T),
                         c_int(inn), c_int(out), c_int(act))
    return y


def skip_layernorm(src, skip, gamma, beta, eps=1e-5):
    src, gamma, beta = _f(src), _f(gamma), _f(beta)
    skip = None if skip is None else _f(skip)
    rows, size = src.shape
    out = np.empty((rows, size), np.float32)
    lib().orc_skip_layernorm(_p(src), _p(skip), _p(gamma), _p(beta), _p(out), c_int(rows),
                             c_int(size), c_float(eps))
    return out


def act(x, kind):
    y = _f(x).copy()
    lib().orc_act(_p(y), c_long(y.size), c_int(kind))
    return y


def attention(q, k, v, batch, seq, nhead, dh_qk, dh_v, mask_kind=0, mask=None, valid_len=None,
              scale=None):
    """q/k/v: 2-D arrays [T, ld]; head h occupies columns h*dh .. (h+1)*dh."""
    q, k, v = _f(q), _f(k), _f(v)
    mask = None if mask is None else _f(mask)
    valid_len = None if valid_len is None else _i(valid_len)
    scale = (1.0 / np.sqrt(dh_qk)) if scale is None else scale
    z = np.empty((batch * seq, nhead * dh_v), np.float32)
    lib().orc_attention(_p(q), _p(k), _p(v), _p(z), c_int(batch), c_int(seq), c_int(nhead),
                        c_int(dh_qk), c_int(dh_v), c_int(q.shape[1]), c_int(k.shape[1]),
                        c_int(v.shape[1]), c_int(nhead * dh_v), c_int(mask_kind), _p(mask),
                        _p(valid_len), c_float(scale))
    return z


def attention_pruned_v(q, k, vc, col_id, head_ptr, batch, seq, nhead, dh_qk, dh_v, mask_kind=0,
                       mask=None, valid_len=None, scale=None):
    q, k, vc = _f(q), _f(k), _f(vc)
    col_id, head_ptr = _i(col_id), _i(head_ptr)
    mask = None if mask is None else _f(mask)
    valid_len = None if valid_len is None else _i(valid_len)
    scale = (1.0 / np.sqrt(dh_qk)) if scale is None else scale
    z = np.empty((batch * seq, nhead * dh_v), np.float32)
    lib().orc_attention_pruned_v(_p(q), _p(k), _p(vc), _p(col_id), _p(head_ptr),
                                 c_int(len(col_id)), _p(z), c_int(batch), c_int(seq),
                                 c_int(nhead), c_int(dh_qk), c_int(dh_v), c_int(q.shape[1]),
                                 c_int(k.shape[1]), c_int(nhead * dh_v), c_int(mask_kind),
                                 _p(mask), _p(valid_len), c_float(scale))
    return z


def fused_vo_attention(q, k, vo, bias_o, batch, seq, nhead, dh_qk, emdim, mask_kind=0, mask=None,
                       valid_len=None, scale=None):
    q, k, vo = _f(q), _f(k), _f(vo)
    bias_o = None if bias_o is None else _f(bias_o)
    mask = None if mask is None else _f(mask)
    valid_len = None if valid_len is None else _i(valid_len)
    scale = (1.0 / np.sqrt(dh_qk)) if scale is None else scale
    out = np.empty((batch * seq, emdim), np.float32)
    lib().orc_fused_vo_attention(_p(q), _p(k), _p(vo), _p(bias_o), _p(out), c_int(batch),
                                 c_int(seq), c_int(nhead), c_int(dh_qk), c_int(emdim),
                                 c_int(q.shape[1]), c_int(k.shape[1]), c_int(mask_kind), _p(mask),
                                 _p(valid_len), c_float(scale))
    return out


def encoder_layer(x, w: dict, batch, seq, nhead, act_kind=2, mask_kind=0, mask=None,
                  valid_len=None, round_mode=0):
    """w: dict of dense arrays as produced by synth.encoder_layer_weights."""
    x = _f(x)
    ws = {k: _f(v) for k, v in w.items()}
    hidden = ws["wo"].shape[0]
    vdim = ws["wo"].shape[1]
    kdim = (ws["wqkv"].shape[0] - vdim) // 2
    ff = ws["w1"].shape[0]
    mask = None if mask is None else _f(mask)
    valid_len = None if valid_len is None else _i(valid_len)
    out = np.empty((batch * seq, hidden), np.float32)
    lib().orc_encoder_layer(_p(x), _p(out), c_int(batch), c_int(seq), c_int(hidden), c_int(nhead),
                            c_int(kdim), c_int(vdim), c_int(ff), _p(ws["wqkv"]), _p(ws["bqkv"]),
                            _p(ws["wo"]), _p(ws["bo"]), _p(ws["w1"]), _p(ws["b1"]), _p(ws["w2"]),
                            _p(ws["b2"]), _p(ws["ln1_g"]), _p(ws["ln1_b"]), _p(ws["ln2_g"]),
                            _p(ws["ln2_b"]), c_int(act_kind), c_int(mask_kind), _p(mask),
                            _p(valid_len), c_int(round_mode))
    return out


def dense_to_tile(W):
    W = _f(W)
    out, inn = W.shape
    n = lib().orc_dense_to_tile(_p(W), c_int(out), c_int(inn), None, None, None)
    row_ptr = np.zeros(out // 16 + 1, np.int32)
    row_off = np.zeros(n, np.int32)
    tiles = np.zeros((n, 256), np.float32)
    lib().orc_dense_to_tile(_p(W), c_int(out), c_int(inn), _p(row_ptr), _p(row_off), _p(tiles))
    return row_ptr, row_off, tiles


def tile_to_dense(row_ptr, row_off, tiles, out, inn):
    W = np.empty((out, inn), np.float32)
    row_ptr, row_off, tiles = _i(row_ptr), _i(row_off), _f(tiles)
    lib().orc_tile_to_dense(_p(row_ptr), _p(row_off), _p(tiles), c_int(out), c_int(inn), _p(W))
    return W


def dense_to_1x16(W):
    W = _f(W)
    out, inn = W.shape
    n = lib().orc_dense_to_1x16(_p(W), c_int(out), c_int(inn), None, None, None)
    tile_idx = np.zeros((out // 16) * (inn // 16 + 1), np.int32)
    row_idx = np.zeros(n, np.int32)
    data = np.zeros((n, 16), np.float32)
    lib().orc_dense_to_1x16(_p(W), c_int(out), c_int(inn), _p(tile_idx), _p(row_idx), _p(data))
    return tile_idx, row_idx, data


def dense_to_csr(W):
    W = _f(W)
    out, inn = W.shape
    n = lib().orc_dense_to_csr(_p(W), c_int(out), c_int(inn), None, None, None)
    indptr = np.zeros(out + 1, np.int32)
    indices = np.zeros(n, np.int32)
    data = np.zeros(n, np.float32)
    lib().orc_dense_to_csr(_p(W), c_int(out), c_int(inn), _p(indptr), _p(indices), _p(data))
    return indptr, indices, data
