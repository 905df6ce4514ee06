"""Runs the C++ driver that exercises the reference-compatible host classes
(scpaper-2021_b200/host/: Linear<MAT>, Attention<config>, Encoder<config>, ...) on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "host_api_test.bin")


@pytest.mark.gpu
def test_cpp_host_api(cuda, orc):
    if not os.path.exists(BIN):
        import __graft_entry__ as entry
        entry.build_cpp_tests()
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=600)
    print(r.stdout[-4000:])
    print(r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-3000:]
    assert "all host-API checks passed" in r.stdout
