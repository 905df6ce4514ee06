"""The shared library loads on a CPU-only box and exports every symbol include/et_b200.h
declares; host-side validators and argument checks work without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "et_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(et_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported(et):
    lib = et.lib()
    declared = _declared()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in et_b200.h but not exported"
    assert sorted(et.ABI_SYMBOLS) == declared


def test_status_strings(et):
    lib = et.lib()
    assert lib.et_status_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.et_status_string(code) not in (b"ok", b"unknown status")
    assert lib.et_built_for_sm() == 100


def test_missing_library_fails_loudly(et, monkeypatch):
    monkeypatch.setattr(et, "_lib", None)
    monkeypatch.setattr(et, "LIB_PATH", "/nonexistent/libet_b200.so")
    with pytest.raises(et.EtError):
        et.lib()


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_validate_tile_mat(et):
    lib = et.lib()
    w = et.synth.prune_tiles(et.synth.normal(1, 1, (64, 96), 1.0), 1, 2, 0.5)
    rp, ro, tiles = et.synth.dense_to_tile(w)
    assert lib.et_validate_tile_mat(_p(rp), _p(ro), len(ro), 96, 64) == 0
    bad = ro.copy()
    bad[0] = 6  # column block out of range (96 / 16 = 6 blocks)
    assert lib.et_validate_tile_mat(_p(rp), _p(bad), len(ro), 96, 64) == -4
    bad = rp.copy()
    bad[1], bad[2] = bad[2], bad[1] if rp[1] != rp[2] else bad[1] + 1
    assert lib.et_validate_tile_mat(_p(bad), _p(ro), len(ro), 96, 64) == -4
    assert lib.et_validate_tile_mat(_p(rp), _p(ro), len(ro) - 1, 96, 64) == -4
    assert lib.et_validate_tile_mat(_p(rp), _p(ro), len(ro), 100, 64) == -3
    assert lib.et_validate_tile_mat(None, _p(ro), len(ro), 96, 64) == -1


def test_validate_lists_1x16_csr(et):
    lib = et.lib()
    ids = np.array([0, 3, 9], np.int32)
    assert lib.et_validate_id_list(_p(ids), 3, 10, 1) == 0
    assert lib.et_validate_id_list(_p(ids), 3, 9, 1) == -4
    assert lib.et_validate_id_list(_p(ids[::-1].copy()), 3, 10, 1) == -4
    assert lib.et_validate_id_list(_p(ids[::-1].copy()), 3, 10, 0) == 0
    w = et.synth.prune_1x16(et.synth.normal(2, 1, (32, 64), 1.0), 2, 2, 0.7)
    ti, ri, data = et.synth.dense_to_1x16(w)
    assert lib.et_validate_1x16(_p(ti), _p(ri), len(ri), 64, 32) == 0
    bad = ri.copy()
    bad[0] += 16
    assert lib.et_validate_1x16(_p(ti), _p(bad), len(ri), 64, 32) == -4
    ip, ix, dv = et.synth.dense_to_csr(w)
    assert lib.et_validate_csr(_p(ip), _p(ix), len(ix), 64, 32) == 0
    bad = ix.copy()
    bad[-1] = 64
    assert lib.et_validate_csr(_p(ip), _p(bad), len(ix), 64, 32) == -4


def test_argument_checks_need_no_gpu(et):
    """Null pointers and bad sizes are refused before any CUDA call."""
    lib = et.lib()
    assert lib.et_linear_dense_fwd(None, None, None, None, 4, 16, 16, 0, None) == -1
    assert lib.et_linear_dense_fwd(None, None, None, None, 4, 20, 16, 0, None) == -3
    assert lib.et_skip_layernorm_fwd(None, None, None, None, None, 1, 8, None) == -1
    assert lib.et_encoder_layer_workspace_bytes(None, 1, 1) == 0


def test_peer_exchange_argument_checks(et):
    """The head-parallel exchange entry points reject bad arguments before touching a device."""
    lib = et.lib()
    lib.et_peer_buffer_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         ctypes.POINTER(ctypes.c_size_t)]
    n = ctypes.c_size_t(0)
    assert lib.et_peer_buffer_bytes(8, 4096, 768, ctypes.byref(n)) == 0
    # partial + y + two output buffers of T x hidden fp16, plus the flag words
    assert n.value >= 4 * 4096 * 768 * 2 and n.value < 4 * 4096 * 768 * 2 + 4096
    assert lib.et_peer_buffer_bytes(17, 4096, 768, ctypes.byref(n)) == -1
    assert lib.et_peer_buffer_bytes(8, 0, 768, ctypes.byref(n)) == -1
    bufs = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    # world out of range, rank out of range, a null buffer, an odd hidden size, misalignment
    assert lib.et_hp_signal_partial_fwd(bufs, 0, 17, 128, 768, 1, None) == -1
    assert lib.et_hp_signal_partial_fwd(bufs, 2, 2, 128, 768, 1, None) == -1
    assert lib.et_hp_signal_partial_fwd((ctypes.c_void_p * 2)(0x1000, None), 0, 2, 128, 768, 1, None) == -1
    assert lib.et_hp_signal_partial_fwd(bufs, 0, 2, 128, 772, 1, None) == -3
    assert lib.et_hp_signal_partial_fwd((ctypes.c_void_p * 2)(0x1000, 0x2010), 0, 2, 128, 768, 1, None) == -2
    assert lib.et_hp_allgather_rows_fwd(bufs, 0, 2, 128, 768, 1, 2, None) == -1
    assert lib.et_peer_buffer_open(None, None) == -1


def test_attention_fuse_o_single_launch_argument_checks(et):
    """The one-kernel attention + output projection rejects bad arguments before touching a
    device (error codes of include/et_b200.h: -1 invalid argument, -2 alignment, -3 shape)."""
    lib = et.lib()
    fn = lib.et_attention_fuse_o_single_launch_fwd
    P = ctypes.c_void_p
    fn.argtypes = [P, P, P, P, P, P, P, P, ctypes.c_int, P, P] + [ctypes.c_int] * 10 + [P, ctypes.c_float, P]
    ok = dict(Q=0x1000, K=0x2000, V=0x3000, mask=None, Z=0x4000, rp=0x5000, ro=0x6000, tiles=0x7000,
              nnz=10, bias=None, out=0x8000, batch=1, seq=128, nhead=12, dh_qk=64, dh_v=64, ldq=768,
              ldk=768, ldv=768, emdim=768, mask_kind=0, vl=None, scale=0.125, stream=None)

    def call(**kw):
        a = dict(ok, **kw)
        return fn(*[a[k] for k in ok])

    assert call(Z=None) == -1 and call(out=None) == -1
    assert call(Q=None) == -1 and call(ro=None) == -1
    assert call(mask_kind=7) == -1
    assert call(mask_kind=2) == -1          # padding mask without lengths
    assert call(scale=0.0) == -1
    assert call(dh_qk=40) == -3             # head width not a multiple of 16
    assert call(ldq=760) == -3              # row pitch narrower than the heads
    assert call(emdim=770) == -3
    assert call(Q=0x1008) == -2

