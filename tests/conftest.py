import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the tests force kernel plans and run instruction-rate probes: load the library build that
# exports the et_debug_* hooks (the product library does not)
os.environ["ET_B200_TEST_HOOKS"] = "1"
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

# fp16-compute tolerance of the hot path against the fp32 oracle
REL_L2_TOL = 5e-3
MAX_ABS_TOL = 2e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def et():
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    o = entry.load_oracle()
    o.build()
    return o


@pytest.fixture(scope="session")
def cuda(et):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    et.lib()
    return torch.device("cuda:0")


def errors(got: np.ndarray, ref: np.ndarray):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    return rel, np.abs(got - ref).max()


def assert_close(got, ref, what="", rel_tol=REL_L2_TOL, abs_tol=MAX_ABS_TOL, dump=None):
    """rel-L2 <= 5e-3 and max-abs <= 2e-2, the tolerance stated for fp16 compute."""
    rel, mx = errors(got, ref)
    dump_dir = os.environ.get("ET_DUMP_DIR")  # set it to keep the arrays of a failing comparison
    if not (rel <= rel_tol and mx <= abs_tol) and dump is not None and dump_dir:
        os.makedirs(dump_dir, exist_ok=True)
        np.savez_compressed(os.path.join(dump_dir, dump + ".npz"),
                            got=np.asarray(got, np.float32), ref=np.asarray(ref, np.float32))
    assert np.isfinite(rel) and rel <= rel_tol and mx <= abs_tol, \
        f"{what}: rel-L2 {rel:.3e} (tol {rel_tol}), max-abs {mx:.3e} (tol {abs_tol})"
