"""The C++ boundary as a drop-in: the reference's own driver sources must compile UNCHANGED
against scpaper-2021_b200/host/ (same include directives, class templates, factories, timers).

The driver files are read from the reference checkout at test time and copied into the
git-ignored build/ directory next to links to our headers, so that their relative includes
(`"../../Fused_attention/Fused_attention.h"`, `<Attention/Attention.h>`, `<wtime.h>` ...) resolve
to this repository's headers.  nvcc -c needs no GPU.  Skipped where the checkout is absent."""
import concurrent.futures
import os
import subprocess

import pytest

import __graft_entry__ as entry

# reference drivers that only use the operator API of the hot path; the ones left out run
# kernels of their own (Linear/test/test_tile.cu, test_outprod.cu: wmma through lib/mma.hpp),
# include kernel internals (Attention/test/test_attn_kernels.cu: ../kernels.h) or call a member
# the reference never defines (Linear/test/test_1x16.cu: forward(float*))
DRIVERS = [
    "test/Table2/main.cu",              # includes template.hpp: test_uniform<>, test_prun_attn1
    "test/main.cu",
    "test/Encoder/test_sparsity.cu",
    "test/Transformer/main.cu",
    "Fused_attention/test/testfused.cu",  # Linear_VO_prune, FusedAttention<NOTF_fused_prune_attn>
    "Fused_attention/test/test_prune.cu",
    "Linear/test/benchmark.cu",          # type_list, make_loop, every Linear<MAT>
    "Linear/test/test_col.cu",
]
EXTRA = ["test/Table2/template.hpp", "test/Transformer/template.hpp"]


@pytest.mark.skipif(not os.path.isdir(entry.REFERENCE_ROOT), reason="reference checkout absent")
def test_reference_drivers_compile_unchanged(tmp_path):
    root = entry.make_dropin_overlay(drivers=DRIVERS + EXTRA)
    # our own instantiation of the template's functions for two weight formats
    own = os.path.join(entry.ROOT, "tests", "cpp", "table2_driver.cu")

    def compile_one(job):
        src, extra = job
        obj = tmp_path / (os.path.basename(src) + "." + str(abs(hash(src)) % 9973) + ".o")
        cmd = [entry.NVCC] + entry.DROPIN_FLAGS + entry.dropin_include_flags() + extra + \
            ["-c", src, "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True, cwd=root)
        return src, r.returncode, (r.stdout + r.stderr)[-3000:]

    jobs = [(os.path.join(root, d), []) for d in DRIVERS]
    jobs.append((own, ["-I" + os.path.join(root, "test", "Table2")]))
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(compile_one, jobs))
    failed = [(s, out) for s, rc, out in results if rc != 0]
    assert not failed, "\n".join(f"{s}:\n{out}" for s, out in failed)
