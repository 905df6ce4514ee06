"""Runs the reference's own paper-table driver (test/Table2/template.hpp, compiled against this
repository's host headers when the library was built) on the GPU: test_uniform<tile_mat>,
test_uniform<base_mat> and test_prun_attn1 must run, and the same configurations with seeded
weights must match the CPU oracle."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "table2_driver.bin")


@pytest.mark.gpu
def test_reference_table2_driver(cuda, orc):
    if not os.path.exists(BIN):
        import __graft_entry__ as entry
        entry.build_cpp_tests()
    if not os.path.exists(BIN):
        pytest.skip("driver not built: it needs the reference checkout at build time")
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=900)
    print(r.stdout[-4000:])
    print(r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-3000:]
    assert "reference Table2 driver: all checks passed" in r.stdout
