"""Generates the golden fixtures under tests/golden/.  Run it where a checkout of the reference
(cctry/SCpaper-2021) is available:

    python tests/golden/make_golden.py <path to the reference checkout>

1. tile_csr_golden.npz   the reference exporter's own tile-CSR builder (gen_csr in
                         example/npy2pt.py:75-109, executed from its source text) applied to
                         seeded matrices: pins the tile-CSR index layout bit-exactly.
2. dense_4_3_csr.bin     output of the reference's mat_type/csr_mat/dense2csr.py for a 4x3
                         matrix: pins the .csr file layout.
3. row_file_golden.bin   a .row file written with the packing rules of
                         mat_type/row_mat/gen_mat.py:17-29 (its compress()).
4. encoder_torch_f64.npz an independent float64 evaluation with PyTorch (nn.functional ops,
                         the framework the reference exports its checkpoints from) of the
                         post-LN encoder layer on seeded inputs: pins the oracle's math.
Inputs are rebuilt from seeds by the tests; only outputs are stored.
"""
import ast
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ET_REFERENCE_DIR", "")
if not os.path.isdir(os.path.join(REF, "example")):
    raise SystemExit("usage: make_golden.py <path to the reference checkout>")
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

et = entry.load_package()


def reference_function(path, name, extra_globals=None):
    """Compiles one top-level function of a reference Python file without importing the file
    (its module-level imports need packages that are not installed here)."""
    tree = ast.parse(open(path).read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name][0]
    mod = ast.Module(body=[fn], type_ignores=[])
    g = {"np": np}
    g.update(extra_globals or {})
    exec(compile(mod, path, "exec"), g)
    return g[name]


def tile_cases():
    cases = {}
    for i, (out, inn, sp) in enumerate([(64, 96, 0.5), (128, 64, 0.8), (48, 48, 0.0), (32, 160, 1.0)]):
        w = et.synth.prune_tiles(et.synth.normal(31, i, (out, inn), 1.0), 31, 100 + i, sp)
        cases[f"case{i}"] = (out, inn, sp, w)
    return cases


def main():
    gen_csr = reference_function(os.path.join(REF, "example", "npy2pt.py"), "gen_csr")
    out = {}
    for name, (o, n, sp, w) in tile_cases().items():
        if sp == 1.0:
            continue  # the exporter cannot represent an all-zero matrix (np.array([]) shapes)
        row_ptr, column, data = gen_csr(w.astype(np.float32))
        out[name + "_row_ptr"], out[name + "_column"], out[name + "_data"] = row_ptr, column, data
    np.savez_compressed(os.path.join(HERE, "tile_csr_golden.npz"), **out)

    with tempfile.TemporaryDirectory() as d:
        subprocess.run([sys.executable, os.path.join(REF, "mat_type", "csr_mat", "dense2csr.py"), "4", "3"],
                       cwd=d, check=True, capture_output=True)
        blob = open(os.path.join(d, "dense_4_3.csr"), "rb").read()
    open(os.path.join(HERE, "dense_4_3_csr.bin"), "wb").write(blob)

    # .row file: compress() of gen_mat.py on a seeded matrix with zeroed rows
    import struct
    nrow, ncol = 32, 16
    mat = et.synth.normal(41, 1, (nrow, ncol), 1.0).astype(np.float64)
    mat[et.synth.choose_ids(41, 2, nrow, 0.5, multiple=1)] = 0
    with tempfile.TemporaryDirectory() as d:
        compress = reference_function(os.path.join(REF, "mat_type", "row_mat", "gen_mat.py"), "compress",
                                      {"struct": struct, "nrow": nrow, "ncol": ncol,
                                       "pack_list": reference_function(os.path.join(REF, "mat_type", "row_mat", "gen_mat.py"), "pack_list", {"struct": struct})})
        cwd = os.getcwd()
        os.chdir(d)
        try:
            compress(mat, "golden")
        finally:
            os.chdir(cwd)
        blob = open(os.path.join(d, "golden.row"), "rb").read()
    open(os.path.join(HERE, "row_file_golden.bin"), "wb").write(blob)

    # float64 PyTorch evaluation of the encoder layer
    import torch
    import torch.nn.functional as F
    res = {}
    for tag, (batch, seq, hidden, nhead, ff, mask_kind) in {
            "c1": (1, 128, 512, 8, 2048, 0),        # BASELINE config 1
            "small_causal": (2, 24, 64, 4, 128, 1),
            "small_padding": (3, 20, 64, 2, 96, 2)}.items():
        w = et.synth.encoder_layer_weights(2021, 0, hidden, ff, bias_std=0.02 if tag != "c1" else 0.0,
                                           ln_noise=0.1 if tag != "c1" else 0.0)
        x = et.synth.normal(2021, 99, (batch * seq, hidden), 1.0)
        t = {k: torch.from_numpy(v.astype(np.float64)) for k, v in w.items()}
        xt = torch.from_numpy(x.astype(np.float64)).reshape(batch, seq, hidden)
        qkv = F.linear(xt, t["wqkv"], t["bqkv"])
        dh = hidden // nhead
        q, k, v = [z.reshape(batch, seq, nhead, dh).transpose(1, 2) for z in qkv.split(hidden, dim=-1)]
        attn_mask = None
        if mask_kind == 1:
            attn_mask = torch.ones(seq, seq, dtype=torch.bool).tril()
        if mask_kind == 2:
            vl = torch.tensor([seq, 7, 1])[:batch]
            attn_mask = (torch.arange(seq)[None, :] < vl[:, None])[:, None, None, :]
        z = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask)
        z = z.transpose(1, 2).reshape(batch, seq, hidden)
        a = F.linear(z, t["wo"], t["bo"])
        y = F.layer_norm(a + xt, (hidden,), t["ln1_g"], t["ln1_b"], 1e-5)
        f = F.gelu(F.linear(y, t["w1"], t["b1"]), approximate="tanh")
        g = F.linear(f, t["w2"], t["b2"])
        o = F.layer_norm(g + y, (hidden,), t["ln2_g"], t["ln2_b"], 1e-5)
        res[tag] = o.reshape(batch * seq, hidden).numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "encoder_torch_f64.npz"), **res)
    print("golden fixtures written")


if __name__ == "__main__":
    main()
