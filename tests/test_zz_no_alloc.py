"""The allocation-free column-pruned Linear (et_linear_col_noalloc_fwd).

Some callers may not allocate device memory at all: a plugin that a host framework hands
nothing but its input and output buffers, or a serving loop that has to stay clear of the
allocator once it is running.  For them the library carries a fixed scratch array of its
own.  This file is collected last so that a run that stops at the first failure has already
been through every other test; it checks the new entry point against the regular one
(et_linear_col_fwd with caller scratch) on two calls in a row, the second with other
inputs and a smaller shape, so stale scratch contents would show."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _case(et, cuda, seed, T, inn, out, sparsity, act):
    x = et.synth.normal(seed, 1, (T, inn), 1.0)
    w = et.synth.normal(seed, 2, (out, inn), 0.05)
    b = et.synth.normal(seed, 3, (out,), 0.1)
    cid, cols = et.synth.dense_to_col(w, et.synth.choose_ids(seed, 4, inn, sparsity))
    return _dev(x, cuda), _dev(cid, cuda), _dev(cols, cuda), _dev(b, cuda), act


def test_noalloc_matches_regular_entry_point_twice(et, cuda):
    import torch
    for seed, T, inn, out, sparsity, act in [(901, 384, 512, 256, 0.5, 1), (902, 130, 256, 128, 0.25, 2)]:
        x, cid, cols, b, act = _case(et, cuda, seed, T, inn, out, sparsity, act)
        ref = et.linear_col(x, cid, cols, b, act)
        y = torch.full((T, out), float("nan"), dtype=torch.float16, device=cuda)
        et.linear_col_noalloc(x, cid, cols, y, b, act)  # warm call: first use of the device
        torch.cuda.synchronize()
        y.fill_(float("nan"))
        torch.cuda.synchronize()
        # the driver's own count of free device memory sees an allocation by ANY route
        # (torch's allocator counter would only see torch's)
        free_before = torch.cuda.mem_get_info()[0]
        before = torch.cuda.memory_allocated()
        et.linear_col_noalloc(x, cid, cols, y, b, act)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        assert et.device_error() == 0
        # same kernels, same operands: the tolerance of the other GPU tests is met with 0 error
        assert torch.equal(y, ref)


def test_noalloc_accepts_exactly_the_builtin_scratch(et, cuda):
    """T * nn_col = 4 194 304 values fills the built-in scratch to the last element."""
    import torch
    T, inn, out = 2048, 2304, 128
    x = _dev(et.synth.normal_fast(903, 1, (T, inn), 1.0), cuda)
    w = et.synth.normal_fast(903, 2, (out, inn), 0.05)
    ids = et.synth.choose_ids(903, 4, inn, 1.0 - 2048 / 2304)
    assert len(ids) == 2048
    cid, cols = et.synth.dense_to_col(w, ids)
    cid, cols = _dev(cid, cuda), _dev(cols, cuda)
    ref = et.linear_col(x, cid, cols, None, 0)
    y = torch.full((T, out), float("nan"), dtype=torch.float16, device=cuda)
    et.linear_col_noalloc(x, cid, cols, y, None, 0)
    torch.cuda.synchronize()
    assert et.device_error() == 0
    assert torch.equal(y, ref)


def test_noalloc_rejects_problems_beyond_the_builtin_scratch(et, cuda):
    import ctypes
    import torch
    x = torch.zeros((16, 16), dtype=torch.float16, device=cuda)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    # T * nn_col = 4 194 304 + 2048 values: refused before anything is launched
    st = et.lib().et_linear_col_noalloc_fwd(vp(x), vp(x), 2048, None, vp(x), vp(x), 2049, 4096, 16,
                                            0, None)
    assert st == -6 and b"scratch" in et.lib().et_status_string(st)
    assert et.device_error() == 0
