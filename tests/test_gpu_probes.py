"""The instruction-rate probes of the hooks library: they run, stay inside their bounded
waits, and report figures in the range the tile-pruned Linear's plan-time choices assume
(a 128 x 16 x 16 tcgen05 product holds the pipe tens of cycles; sixteen mma.sync.m16n8k16 per
tile sustain several hundred multiply-accumulates per clock and SM)."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


def test_tcgen05_narrow_product_cost(et, cuda):
    L = et.lib()
    out = ctypes.c_double(0.0)
    # N = 16 and N = 256, 128 rows, four accumulators, 2048 products back to back
    assert L.et_debug_probe_tcgen05(128, 16, 4, 2048, 1, ctypes.byref(out)) == 0
    narrow = out.value
    assert L.et_debug_probe_tcgen05(128, 256, 2, 2048, 1, ctypes.byref(out)) == 0
    wide = out.value
    assert et.device_error() == 0
    # the narrow product costs far more than its share of the arithmetic (16 / 256 of wide)
    assert 20.0 < narrow < 120.0, narrow
    assert 100.0 < wide < 200.0, wide
    assert narrow > 3.0 * wide * 16 / 256


@pytest.mark.parametrize("mode", [0, 1])
def test_mma_sync_rate(et, cuda, mode):
    L = et.lib()
    out = ctypes.c_double(0.0)
    assert L.et_debug_probe_mma_sync(8, 2, 2000, mode, ctypes.byref(out)) == 0
    assert et.device_error() == 0
    assert 400.0 < out.value < 2100.0, out.value


def test_mixed_paths_share_the_pipe(et, cuda):
    L = et.lib()
    cyc, mac = ctypes.c_double(0.0), ctypes.c_double(0.0)
    assert L.et_debug_probe_mixed(4, 2048, 8, 2000, 0, ctypes.byref(cyc), ctypes.byref(mac)) == 0
    both_mac = mac.value
    assert L.et_debug_probe_mixed(1, 0, 8, 2000, 0, ctypes.byref(cyc), ctypes.byref(mac)) == 0
    solo_mac = mac.value
    assert et.device_error() == 0
    assert solo_mac > 400.0
    assert both_mac < solo_mac  # the warp-level path slows down while tcgen05 products run
