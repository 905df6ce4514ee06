"""Weight import / export and inference-time preparation of pruned checkpoints (host code).

On-disk formats are the reference's own:

* one `.npz` per parameter group, written by its exporter (example/npy2pt.py:112-119) and read
  by its example driver (example/main.cu:44-100): 2-D weights as tile-CSR with keys `row_ptr`
  (int32), `column` (int32), `data` (float32 [nnz, 256]) and `B` (float32 bias); LayerNorm
  parameters as `W`, `B`; file names `transformer_encoder.layers.<l>.<group>.npz` with the
  groups `self_attn.in_proj_`, `self_attn.out_proj.`, `linear1.`, `linear2.`, `norm1.`,
  `norm2.`, and a `weights.txt` that lists them;
* raw `.row` / `.col` files (mat_type/row_mat/row_mat.hpp:15-29, mat_type/col_mat/col_mat.hpp:
  22-36, writer mat_type/row_mat/gen_mat.py:17-29): `uint32 nrow, ncol, len; uint32 ids[len];
  float32 values[...]`;
* raw `.csr` files (mat_type/csr_mat/csr_mat.h:19-35): `uint32 nrow, ncol, nnz; int32
  indptr[nrow + 1]; int32 indices[nnz]; float32 data[nnz]`.

Plus the two preparation steps the reference leaves to "elsewhere": the pre-multiplied per-head
V.O weight of the fused attention (Fused_attention/Linear_VO.h:22-47) and magnitude-based
selection of what to prune (the reference's pruning submodule is empty).
"""
from __future__ import annotations

import os
import struct

import numpy as np

from . import synth

GROUPS = {"wqkv": "self_attn.in_proj_", "wo": "self_attn.out_proj.", "w1": "linear1.",
          "w2": "linear2.", "ln1": "norm1.", "ln2": "norm2."}
BIAS_OF = {"wqkv": "bqkv", "wo": "bo", "w1": "b1", "w2": "b2"}


def layer_file(folder: str, layer: int, group: str) -> str:
    return os.path.join(folder, f"transformer_encoder.layers.{layer}.{GROUPS[group]}.npz")


# ---- .npz (tile-CSR) ---------------------------------------------------------------------

def save_tile_npz(path: str, W: np.ndarray, bias: np.ndarray) -> None:
    """2-D weight -> the exporter's tile-CSR .npz (all-zero tiles dropped)."""
    row_ptr, row_off, tiles = synth.dense_to_tile(np.asarray(W, np.float32))
    np.savez(path, row_ptr=row_ptr.astype(np.int32), column=row_off.astype(np.int32),
             data=tiles.reshape(-1, 256).astype(np.float32), B=np.asarray(bias, np.float32))


def load_tile_npz(path: str):
    """-> (row_ptr int32, row_off int32, tiles fp16 [nnz, 256], bias fp16).  Index arrays are
    checked for the invariants the kernels rely on."""
    z = np.load(path)
    row_ptr = np.asarray(z["row_ptr"], np.int32)
    row_off = np.asarray(z["column"], np.int32).reshape(-1)
    tiles = np.asarray(z["data"], np.float32).reshape(-1, 256)
    bias = np.asarray(z["B"], np.float32).reshape(-1)
    if row_ptr.ndim != 1 or len(row_ptr) < 2 or row_ptr[0] != 0 or row_ptr[-1] != len(row_off):
        raise ValueError(f"{path}: row_ptr does not describe {len(row_off)} tiles")
    if np.any(np.diff(row_ptr) < 0) or len(tiles) != len(row_off):
        raise ValueError(f"{path}: inconsistent tile-CSR arrays")
    if len(bias) != (len(row_ptr) - 1) * 16:
        raise ValueError(f"{path}: bias length {len(bias)} != 16 x block rows")
    return row_ptr, row_off, tiles.astype(np.float16), bias.astype(np.float16)


def save_norm_npz(path: str, gamma: np.ndarray, beta: np.ndarray) -> None:
    np.savez(path, W=np.asarray(gamma, np.float32), B=np.asarray(beta, np.float32))


def load_norm_npz(path: str):
    z = np.load(path)
    return np.asarray(z["W"], np.float32).astype(np.float16), \
        np.asarray(z["B"], np.float32).astype(np.float16)


def save_layer(folder: str, layer: int, w: dict) -> list[str]:
    """Writes one encoder layer (dict as synth.encoder_layer_weights returns) in the exporter's
    layout; returns the file names (the lines of weights.txt)."""
    os.makedirs(folder, exist_ok=True)
    names = []
    for key in ("wqkv", "wo", "w1", "w2"):
        p = layer_file(folder, layer, key)
        save_tile_npz(p, w[key], w[BIAS_OF[key]])
        names.append(os.path.basename(p))
    for key in ("ln1", "ln2"):
        p = layer_file(folder, layer, key)
        save_norm_npz(p, w[key + "_g"], w[key + "_b"])
        names.append(os.path.basename(p))
    with open(os.path.join(folder, "weights.txt"), "a") as f:
        f.writelines(n + "\n" for n in names)
    return names


def load_layer(folder: str, layer: int, in_sizes: dict) -> dict:
    """Reads one layer back as dense fp16 arrays (the dict EncoderLayer takes).  `in_sizes`
    gives the input width of each weight ({"wqkv": hidden, "wo": vdim, "w1": hidden, "w2": ff}):
    tile-CSR does not store it (the reference passes it to tile_mat's constructor)."""
    w = {}
    for key in ("wqkv", "wo", "w1", "w2"):
        rp, ro, tiles, bias = load_tile_npz(layer_file(folder, layer, key))
        out = (len(rp) - 1) * 16
        inn = int(in_sizes[key])
        if len(ro) and (ro.min() < 0 or ro.max() >= inn // 16):
            raise ValueError(f"{key}: tile column outside [0, {inn // 16})")
        w[key] = synth.tile_to_dense(rp, ro, tiles, out, inn)
        w[BIAS_OF[key]] = bias
    for key in ("ln1", "ln2"):
        w[key + "_g"], w[key + "_b"] = load_norm_npz(layer_file(folder, layer, key))
    return w


# ---- raw .row / .col / .csr --------------------------------------------------------------

def write_row_file(path: str, nrow: int, row_id: np.ndarray, rows: np.ndarray) -> None:
    rows = np.asarray(rows, np.float32)
    with open(path, "wb") as f:
        f.write(struct.pack("III", nrow, rows.shape[1], len(row_id)))
        f.write(np.asarray(row_id, np.uint32).tobytes())
        f.write(rows.tobytes())


def read_row_file(path: str):
    """-> (nrow, row_id int32 [len], rows float32 [len, ncol])."""
    blob = open(path, "rb").read()
    nrow, ncol, n = struct.unpack_from("III", blob, 0)
    if len(blob) != 12 + 4 * n + 4 * n * ncol:
        raise ValueError(f"{path}: size does not match its header")
    ids = np.frombuffer(blob, np.uint32, n, 12).astype(np.int32)
    rows = np.frombuffer(blob, np.float32, n * ncol, 12 + 4 * n).reshape(n, ncol).copy()
    if n and (ids.max() >= nrow or np.any(np.diff(ids) <= 0)):
        raise ValueError(f"{path}: row ids must be ascending and below {nrow}")
    return nrow, ids, rows


def write_col_file(path: str, ncol: int, col_id: np.ndarray, cols: np.ndarray) -> None:
    """cols: [nrow, len] (the kept input columns of a [nrow, ncol] matrix)."""
    cols = np.asarray(cols, np.float32)
    with open(path, "wb") as f:
        f.write(struct.pack("III", cols.shape[0], ncol, len(col_id)))
        f.write(np.asarray(col_id, np.uint32).tobytes())
        f.write(cols.tobytes())


def read_col_file(path: str):
    """-> (ncol, col_id int32 [len], cols float32 [nrow, len])."""
    blob = open(path, "rb").read()
    nrow, ncol, n = struct.unpack_from("III", blob, 0)
    if len(blob) != 12 + 4 * n + 4 * n * nrow:
        raise ValueError(f"{path}: size does not match its header")
    ids = np.frombuffer(blob, np.uint32, n, 12).astype(np.int32)
    cols = np.frombuffer(blob, np.float32, n * nrow, 12 + 4 * n).reshape(nrow, n).copy()
    if n and ids.max() >= ncol:
        raise ValueError(f"{path}: column id outside [0, {ncol})")
    return ncol, ids, cols


def write_csr_file(path: str, W: np.ndarray) -> None:
    indptr, indices, data = synth.dense_to_csr(np.asarray(W, np.float32))
    with open(path, "wb") as f:
        f.write(struct.pack("III", W.shape[0], W.shape[1], len(data)))
        f.write(indptr.astype(np.int32).tobytes())
        f.write(indices.astype(np.int32).tobytes())
        f.write(data.astype(np.float32).tobytes())


def read_csr_file(path: str):
    """-> (nrow, ncol, indptr, indices, data float32)."""
    blob = open(path, "rb").read()
    nrow, ncol, nnz = struct.unpack_from("III", blob, 0)
    if len(blob) != 12 + 4 * (nrow + 1) + 8 * nnz:
        raise ValueError(f"{path}: size does not match its header")
    indptr = np.frombuffer(blob, np.int32, nrow + 1, 12).copy()
    indices = np.frombuffer(blob, np.int32, nnz, 12 + 4 * (nrow + 1)).copy()
    data = np.frombuffer(blob, np.float32, nnz, 12 + 4 * (nrow + 1) + 4 * nnz).copy()
    if indptr[0] != 0 or indptr[-1] != nnz or np.any(np.diff(indptr) < 0):
        raise ValueError(f"{path}: bad indptr")
    if nnz and (indices.min() < 0 or indices.max() >= ncol):
        raise ValueError(f"{path}: column index outside [0, {ncol})")
    return nrow, ncol, indptr, indices, data


# ---- fused V.O weights -------------------------------------------------------------------

def build_w_vo(wv: np.ndarray, bv, wo: np.ndarray, nhead: int):
    """Pre-multiplies the V and O projections per head (fp32 arithmetic, fp16 result):
    W_VO[h] = Wv_h^T . Wo_h^T  [emdim_in, emdim_out]  so that  VO_h = X . W_VO[h]  and the
    attention output is  sum_h P_h . VO_h + b_O  (layout of Fused_attention/Linear_VO.h:42-47).
    The V bias folds into a per-head output bias  b_VO[h] = bv_h . Wo_h^T  (rows of P sum to 1).
    wv: [vdim, emdim_in], wo: [emdim_out, vdim].  -> (w_vo fp16 [nhead, in, out],
    b_vo fp16 [nhead, out])."""
    wv = np.asarray(wv, np.float32)
    wo = np.asarray(wo, np.float32)
    vdim, emdim_in = wv.shape
    if wo.shape[1] != vdim or vdim % nhead:
        raise ValueError("wv / wo shapes do not match nhead")
    dv = vdim // nhead
    bv = np.zeros(vdim, np.float32) if bv is None else np.asarray(bv, np.float32)
    w_vo = np.empty((nhead, emdim_in, wo.shape[0]), np.float32)
    b_vo = np.empty((nhead, wo.shape[0]), np.float32)
    for h in range(nhead):
        wo_h = wo[:, h * dv:(h + 1) * dv]              # [out, dv]
        w_vo[h] = wv[h * dv:(h + 1) * dv].T @ wo_h.T   # [in, dv] . [dv, out]
        b_vo[h] = bv[h * dv:(h + 1) * dv] @ wo_h.T
    return w_vo.astype(np.float16), b_vo.astype(np.float16)


# ---- magnitude-based selection -----------------------------------------------------------

def _keep_largest(score: np.ndarray, sparsity: float) -> np.ndarray:
    """Boolean mask keeping the round((1 - sparsity) * n) largest scores (ties: lower index)."""
    n = score.size
    keep = int(round((1.0 - sparsity) * n))
    order = np.argsort(-score.reshape(-1), kind="stable")
    mask = np.zeros(n, bool)
    mask[order[:keep]] = True
    return mask.reshape(score.shape)


def magnitude_prune_tiles(W: np.ndarray, sparsity: float) -> np.ndarray:
    """Zeroes the 16x16 tiles of smallest L2 norm (the tile_mat granularity)."""
    out, inn = W.shape
    t = np.asarray(W, np.float32).reshape(out // 16, 16, inn // 16, 16)
    m = _keep_largest((t * t).sum(axis=(1, 3)), sparsity)
    return (t * m[:, None, :, None]).reshape(out, inn).astype(W.dtype)


def magnitude_prune_1x16(W: np.ndarray, sparsity: float) -> np.ndarray:
    """Zeroes the 1x16 vectors (one output row, 16 consecutive inputs) of smallest L2 norm."""
    out, inn = W.shape
    t = np.asarray(W, np.float32).reshape(out, inn // 16, 16)
    m = _keep_largest((t * t).sum(axis=2), sparsity)
    return (t * m[:, :, None]).reshape(out, inn).astype(W.dtype)


def magnitude_select_rows(W: np.ndarray, sparsity: float, multiple: int = 16) -> np.ndarray:
    """Sorted ids of the output rows to keep (largest L2 norm), count rounded down to a
    multiple of `multiple` as the reference pads its id lists (row_mat.cu:5-25)."""
    score = (np.asarray(W, np.float32) ** 2).sum(axis=1)
    keep = int(np.floor(len(score) * (1.0 - sparsity) + 1e-9)) // multiple * multiple
    return np.sort(np.argsort(-score, kind="stable")[:keep]).astype(np.int32)


def magnitude_select_cols(W: np.ndarray, sparsity: float, multiple: int = 16) -> np.ndarray:
    """Sorted ids of the input columns to keep (largest L2 norm)."""
    return magnitude_select_rows(np.asarray(W).T, sparsity, multiple)
