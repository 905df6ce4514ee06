"""Compiles the reference's OWN CUDA implementation of the encoder path for sm_100a, straight
from the sources where they lie in the reference checkout, with nvcc (the reference's CMake
build is not run), and links it with a small driver of ours into oracle/_ref/ref_table2.

    python oracle/ref_cuda/build_ref_cuda.py [reference root]

The binary is a reported baseline ("the reference's own CUDA build, recompiled"), never an
oracle: its outputs are not compared with anything.  oracle/_ref/ is git-ignored; no reference
source is copied into the repository.  Needs cuBLAS and cuSPARSE from the CUDA toolkit.
Flags follow the reference's top-level CMakeLists.txt (relaxed constexpr, extended lambdas,
per-thread default stream, OpenMP host flag), the architecture is 100a instead of 70.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "_ref")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

SOURCES = [
    "lib/utils.cu", "lib/CUDA_ptr.cu", "mycublas/cublas.cu",
    "mat_type/tile_mat/tile_mat.cu", "mat_type/row_mat/row_mat.cu", "mat_type/col_mat/col_mat.cu",
    "mat_type/mat1x16/mat1x16.cu", "mat_type/csr_mat/csr_mat.cpp",
    "Linear/Linear.cu", "Linear/SPMM_tile.cu", "Linear/SPMM_row.cu", "Linear/SPMM_col.cu",
    "Linear/cusp.cu", "Linear/SPMM1x16.cu",
    "Attention/Attention.cu", "Attention/kernels.cu", "Attention/prune_attn.cu",
    "Attention/mixed-precision/mixed_attn.cu", "Attention/kernel_fuseO.cu",
    "Attention/Attention_single.cu",
    "SkipLayerNorm/SkipLayerNorm.cu", "LayerNorm/LayerNorm.cu", "Encoder/Encoder.cu",
    "Fused_attention/Fused_attention.cu", "Fused_attention/Linear_VO.cu",
]


def build(ref_root: str = "/root/reference") -> str:
    if not os.path.isdir(ref_root):
        raise FileNotFoundError(ref_root)
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(os.path.dirname(os.path.dirname(HERE)), "build", "ref_cuda")
    os.makedirs(obj_dir, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-ccbin", "/usr/bin/g++",
             "--expt-relaxed-constexpr", "--extended-lambda", "--default-stream", "per-thread",
             "-Xcompiler", "-fopenmp", "-w", "-x", "cu",
             "-I" + ref_root, "-I" + os.path.join(ref_root, "lib"),
             "-I" + os.path.join(ref_root, "mycublas"), "-I" + os.path.join(ref_root, "mat_type")]

    def compile_one(rel: str) -> str:
        obj = os.path.join(obj_dir, rel.replace("/", "_") + ".o")
        src = os.path.join(ref_root, rel)
        if not os.path.exists(obj) or os.path.getmtime(src) > os.path.getmtime(obj):
            r = subprocess.run([NVCC] + flags + ["-c", src, "-o", obj], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {rel}:\n{r.stdout}{r.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    driver = os.path.join(HERE, "table2_ref_driver.cu")
    drv_obj = os.path.join(obj_dir, "driver.o")
    r = subprocess.run([NVCC] + flags + ["-I" + os.path.join(ref_root, "test", "Table2"), "-c", driver,
                                         "-o", drv_obj], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on the driver:\n{r.stdout}{r.stderr}")
    out = os.path.join(OUT_DIR, "ref_table2")
    r = subprocess.run([NVCC, "-ccbin", "/usr/bin/g++", "-gencode", "arch=compute_100a,code=sm_100a",
                        "-Xcompiler", "-fopenmp", "-o", out, drv_obj] + objs + ["-lcublas", "-lcusparse"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return out


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
