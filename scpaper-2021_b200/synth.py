"""Seeded synthetic tensors and pruned-weight format builders (host side, numpy).

The generator is counter based: element i of tensor `tensor_id` under `seed` depends only on
(seed, tensor_id, i), so any rank or process can rebuild any slice without communication.
SplitMix64 supplies the bits, Box-Muller the normal deviates; values are rounded to fp16,
the storage type of the GPU path.

The format builders follow the reference's containers:
  tile-CSR   mat_type/tile_mat/tile_mat.h:36-45, example/npy2pt.py:75-109
  row / col  mat_type/row_mat/row_mat.hpp:9-56, mat_type/col_mat/col_mat.hpp:10-73
  1x16       mat_type/mat1x16/mat1x16.h:5-22
  CSR        mat_type/csr_mat/csr_mat.h:11-42
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _key(seed: int, tensor_id: int) -> np.uint64:
    k = _splitmix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))
    k = _splitmix64(k ^ np.uint64(tensor_id & 0xFFFFFFFFFFFFFFFF))
    return k[0]


def uniform(seed: int, tensor_id: int, n: int, offset: int = 0, stream: int = 0) -> np.ndarray:
    """n doubles in (0, 1): elements offset .. offset + n of the tensor's stream."""
    idx = np.arange(offset, offset + n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        ctr = (idx * np.uint64(2) + np.uint64(stream)) & _M64
        bits = _splitmix64(ctr ^ _key(seed, tensor_id))
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))


def normal(seed: int, tensor_id: int, shape, std: float = 1.0, mean: float = 0.0) -> np.ndarray:
    """fp16-rounded N(mean, std^2) values, returned as float16."""
    n = int(np.prod(shape))
    u1 = uniform(seed, tensor_id, n, stream=0)
    u2 = uniform(seed, tensor_id, n, stream=1)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).astype(np.float32).astype(np.float16).reshape(shape)


def permutation(seed: int, tensor_id: int, n: int) -> np.ndarray:
    """A seeded permutation of range(n) (stable argsort of counter-based keys)."""
    return np.argsort(uniform(seed, tensor_id, n), kind="stable")


def keep_exact(seed: int, tensor_id: int, n: int, sparsity: float) -> np.ndarray:
    """Boolean keep-mask over n units with exactly floor(n * (1 - sparsity)) kept, the count
    rule of the reference's generators (mat_type/tile_mat/tile_mat.cu:12-17)."""
    keep = int(np.floor(n * (1.0 - sparsity) + 1e-9))
    m = np.zeros(n, dtype=bool)
    m[permutation(seed, tensor_id, n)[:keep]] = True
    return m


# ---------------------------------------------------------------------------------------
# pruning masks
# ---------------------------------------------------------------------------------------

def prune_tiles(W: np.ndarray, seed: int, tensor_id: int, sparsity: float) -> np.ndarray:
    """Zeroes 16x16 tiles of W[out, in] uniformly at random (exact count)."""
    out, inn = W.shape
    m = keep_exact(seed, tensor_id, (out // 16) * (inn // 16), sparsity).reshape(out // 16, inn // 16)
    return W * np.kron(m, np.ones((16, 16), dtype=bool)).astype(W.dtype)


def prune_1x16(W: np.ndarray, seed: int, tensor_id: int, sparsity: float) -> np.ndarray:
    """Zeroes 1x16 vectors (one output row, 16 consecutive inputs) uniformly at random."""
    out, inn = W.shape
    m = keep_exact(seed, tensor_id, out * (inn // 16), sparsity).reshape(out, inn // 16)
    return W * np.repeat(m, 16, axis=1).astype(W.dtype)


def choose_ids(seed: int, tensor_id: int, n: int, sparsity: float, multiple: int = 16) -> np.ndarray:
    """Sorted kept indices out of range(n): floor(n * (1 - sparsity)) rounded down to a
    multiple of `multiple` (the reference pads its id lists to x16, row_mat.cu:5-25)."""
    keep = int(np.floor(n * (1.0 - sparsity) + 1e-9)) // multiple * multiple
    return np.sort(permutation(seed, tensor_id, n)[:keep]).astype(np.int32)


# ---------------------------------------------------------------------------------------
# dense <-> format converters (index handling is integer exact)
# ---------------------------------------------------------------------------------------

def dense_to_tile(W: np.ndarray):
    """Dense [out, in] -> (row_ptr, row_off, tiles[nnz, 256]).  A tile is dropped iff all of
    its 256 values are exactly zero; order is block-row-major, then block column."""
    out, inn = W.shape
    assert out % 16 == 0 and inn % 16 == 0
    nbr, nbc = out // 16, inn // 16
    blocks = W.reshape(nbr, 16, nbc, 16).transpose(0, 2, 1, 3)  # [nbr, nbc, 16, 16]
    present = (blocks != 0).any(axis=(2, 3))
    row_ptr = np.zeros(nbr + 1, dtype=np.int32)
    row_ptr[1:] = np.cumsum(present.sum(axis=1))
    br, bc = np.nonzero(present)
    tiles = blocks[br, bc].reshape(-1, 256).astype(W.dtype)
    return row_ptr, bc.astype(np.int32), np.ascontiguousarray(tiles)


def tile_to_dense(row_ptr, row_off, tiles, out: int, inn: int) -> np.ndarray:
    W = np.zeros((out, inn), dtype=tiles.dtype)
    for br in range(out // 16):
        for i in range(row_ptr[br], row_ptr[br + 1]):
            c = int(row_off[i]) * 16
            W[br * 16:br * 16 + 16, c:c + 16] = tiles[i].reshape(16, 16)
    return W


def dense_to_row(W: np.ndarray, row_id: np.ndarray):
    """Kept output rows: (row_id, rows[nn_row, in])."""
    return row_id.astype(np.int32), np.ascontiguousarray(W[row_id])


def dense_to_col(W: np.ndarray, col_id: np.ndarray):
    """Kept input columns: (col_id, cols[out, nn_col])."""
    return col_id.astype(np.int32), np.ascontiguousarray(W[:, col_id])


def dense_to_1x16(W: np.ndarray):
    """Dense -> (tile_idx[(out/16) * (in/16 + 1)], row_idx[nvec], data[nvec, 16]).  A vector is
    dropped iff its 16 values are all zero; inside a (row set, part) group vectors are stored
    by ascending row; row_idx holds the global output row."""
    out, inn = W.shape
    nset, npart = out // 16, inn // 16
    vec = W.reshape(nset, 16, npart, 16)                      # [set, q, part, 16]
    present = (vec != 0).any(axis=3).transpose(0, 2, 1)       # [set, part, q]
    counts = present.sum(axis=2)                              # [set, part]
    tile_idx = np.zeros((nset, npart + 1), dtype=np.int32)
    run = 0
    for r in range(nset):
        tile_idx[r, 0] = run
        tile_idx[r, 1:] = run + np.cumsum(counts[r])
        run = int(tile_idx[r, npart])
    s, p, q = np.nonzero(present)
    row_idx = (s * 16 + q).astype(np.int32)
    data = vec[s, q, p].astype(W.dtype)
    return tile_idx.reshape(-1), row_idx, np.ascontiguousarray(data.reshape(-1, 16))


def dense_to_csr(W: np.ndarray):
    out, _ = W.shape
    nz = W != 0
    indptr = np.zeros(out + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(nz.sum(axis=1))
    r, c = np.nonzero(nz)
    return indptr, c.astype(np.int32), np.ascontiguousarray(W[r, c])


def head_ptr_for(col_id: np.ndarray, nhead: int, vdim: int) -> np.ndarray:
    """head_ptr[h] .. head_ptr[h+1]: entries of the sorted col_id list that fall in head h
    (mat_type/col_mat/col_mat.cu:34-58)."""
    dh = vdim // nhead
    return np.searchsorted(col_id, np.arange(nhead + 1) * dh, side="left").astype(np.int32)


# ---------------------------------------------------------------------------------------
# encoder-layer weights
# ---------------------------------------------------------------------------------------

def normal_fast(seed: int, tensor_id: int, shape, std: float = 1.0, mean: float = 0.0) -> np.ndarray:
    """N(mean, std^2) fp16 values from numpy's PCG64 keyed by (seed, tensor_id): an order of
    magnitude faster than the counter-based generator, for large benchmark-only tensors whose
    values nothing else has to reproduce element by element."""
    rng = np.random.Generator(np.random.PCG64([int(seed) & 0xFFFFFFFF, int(tensor_id) & 0xFFFFFFFF]))
    v = rng.standard_normal(int(np.prod(shape)), dtype=np.float32)
    return (v * np.float32(std) + np.float32(mean)).astype(np.float16).reshape(shape)


def encoder_layer_weights(seed: int, layer: int, hidden: int, ff: int, kdim: int | None = None,
                          vdim: int | None = None, std: float = 0.02, bias_std: float = 0.0,
                          ln_noise: float = 0.0, fast: bool = False) -> dict:
    """Dense fp16 weights of one post-LN encoder layer: W ~ N(0, std^2), biases 0 (or
    N(0, bias_std^2)), LN gamma 1 and beta 0 (plus optional noise so tests exercise them).
    wqkv has its output features ordered Q | K | V.  fast=True draws from normal_fast."""
    kdim = hidden if kdim is None else kdim
    vdim = hidden if vdim is None else vdim
    base = 1000 * (layer + 1)
    normal = normal_fast if fast else globals()["normal"]
    def b(tid, n):
        return normal(seed, base + tid, (n,), bias_std) if bias_std > 0 else np.zeros(n, np.float16)
    w = {
        "wqkv": normal(seed, base + 1, (2 * kdim + vdim, hidden), std),
        "bqkv": b(2, 2 * kdim + vdim),
        "wo": normal(seed, base + 3, (hidden, vdim), std),
        "bo": b(4, hidden),
        "w1": normal(seed, base + 5, (ff, hidden), std),
        "b1": b(6, ff),
        "w2": normal(seed, base + 7, (hidden, ff), std),
        "b2": b(8, hidden),
    }
    for i, name in enumerate(("ln1", "ln2")):
        if ln_noise > 0:
            w[name + "_g"] = normal(seed, base + 9 + 2 * i, (hidden,), ln_noise, 1.0)
            w[name + "_b"] = normal(seed, base + 10 + 2 * i, (hidden,), ln_noise, 0.0)
        else:
            w[name + "_g"] = np.ones(hidden, np.float16)
            w[name + "_b"] = np.zeros(hidden, np.float16)
    return w


def mixed_format_layer(seed: int, layer: int, hidden: int, ff: int, vec_sparsity: float = 0.9,
                       ffn_sparsity: float = 0.5, **kw):
    """One encoder layer pruned the way the paper's BERT-large configuration is: Q/K/V and O
    projections as 1x16 vectors (`vec_sparsity` of them dropped), FFN hidden units pruned
    (`ffn_sparsity`): the first FFN Linear keeps those output rows, the second reads exactly
    those input columns.  Returns (weights, formats): `weights` are the dense equivalents
    (pruned entries zero) the CPU oracle evaluates, `formats` the per-weight storage formats
    for EncoderLayer (the row and column lists are one array object)."""
    w = encoder_layer_weights(seed, layer, hidden, ff, **kw)
    base = 1000 * (layer + 1)
    w["wqkv"] = prune_1x16(w["wqkv"], seed, base + 60, vec_sparsity)
    w["wo"] = prune_1x16(w["wo"], seed, base + 61, vec_sparsity)
    ids = choose_ids(seed, base + 62, ff, ffn_sparsity)
    keep = np.zeros(ff, dtype=bool)
    keep[ids] = True
    w["w1"] = np.where(keep[:, None], w["w1"], np.float16(0)).astype(np.float16)
    w["w2"] = np.where(keep[None, :], w["w2"], np.float16(0)).astype(np.float16)
    formats = {"wqkv": "1x16_auto", "wo": "1x16_auto", "w1": ("row", ids), "w2": ("col", ids)}
    return w, formats
