"""GPU parity of SkipLayerNorm / LayerNorm / activation / bias passes against the oracle."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("rows,size", [(1, 8), (7, 768), (2048, 768), (130, 1024), (5, 4096),
                                       (3, 2056)])
def test_skip_layernorm(et, orc, cuda, rows, size):
    src = et.synth.normal(5, 1, (rows, size), 2.0, 0.5)
    skip = et.synth.normal(5, 2, (rows, size), 1.0)
    g = et.synth.normal(5, 3, (size,), 0.2, 1.0)
    b = et.synth.normal(5, 4, (size,), 0.2)
    y = et.skip_layernorm(_dev(src, cuda), _dev(skip, cuda), _dev(g, cuda), _dev(b, cuda))
    assert_close(y.float().cpu().numpy(), orc.skip_layernorm(src, skip, g, b), "skipLN")
    y = et.layernorm(_dev(src, cuda), _dev(g, cuda), _dev(b, cuda))
    assert_close(y.float().cpu().numpy(), orc.skip_layernorm(src, None, g, b), "LN")


def test_layernorm_constant_row(et, cuda):
    """A constant row normalises to beta (gamma = beta = 0.2: SkipLayerNorm.cu:84-89)."""
    import torch
    src = torch.full((4, 768), 0.2, dtype=torch.float16, device=cuda)
    g = torch.full((768,), 0.2, dtype=torch.float16, device=cuda)
    y = et.layernorm(src, g, g)
    assert torch.allclose(y.float(), torch.full_like(y, 0.2).float(), atol=2e-3)


@pytest.mark.parametrize("kind", [1, 2])
@pytest.mark.parametrize("n", [8, 1000, 128 * 3072 + 3])
def test_act(et, orc, cuda, kind, n):
    x = et.synth.normal(6, 1, (n,), 2.0)
    y = et.act(_dev(x, cuda), kind)
    assert_close(y.float().cpu().numpy(), orc.act(x, kind), f"act {kind}")
    xi = _dev(x, cuda)
    et.act(xi, kind, inplace=True)
    assert_close(xi.float().cpu().numpy(), orc.act(x, kind), f"act in place {kind}")


def test_bias_add(et, cuda):
    x = et.synth.normal(7, 1, (33, 64), 1.0)
    b = et.synth.normal(7, 2, (64,), 1.0)
    y = et.bias_add_(_dev(x, cuda), _dev(b, cuda))
    ref = (x.astype(np.float32) + b.astype(np.float32)).astype(np.float16).astype(np.float32)
    assert np.array_equal(y.float().cpu().numpy(), ref)


@pytest.mark.parametrize("T,inn,out", [(2048, 768, 768), (300, 256, 256), (130, 3072, 768),
                                       (100, 512, 1024), (1, 64, 384), (257, 1024, 1024),
                                       (70, 80, 256), (129, 16, 640)])
@pytest.mark.parametrize("with_bias,with_resid", [(True, True), (False, True), (True, False)])
def test_linear_skip_layernorm(et, orc, cuda, T, inn, out, with_bias, with_resid):
    """Dense Linear + residual + LayerNorm in one kernel (a cluster of out / 128 CTAs per row
    block) against the oracle's Linear followed by its SkipLayerNorm."""
    x = et.synth.normal(8, 1, (T, inn), 1.0)
    w = et.synth.normal(8, 2, (out, inn), 0.05)
    b = et.synth.normal(8, 3, (out,), 0.5) if with_bias else None
    res = et.synth.normal(8, 4, (T, out), 1.0, 0.3) if with_resid else None
    g = et.synth.normal(8, 5, (out,), 0.2, 1.0)
    beta = et.synth.normal(8, 6, (out,), 0.2)
    y = et.linear_skip_layernorm(_dev(x, cuda), _dev(w, cuda),
                                 _dev(b, cuda) if with_bias else None,
                                 _dev(res, cuda) if with_resid else None, _dev(g, cuda),
                                 _dev(beta, cuda))
    assert et.device_error() == 0
    ref = orc.skip_layernorm(orc.linear_dense(x, w, b, 0), res, g, beta)
    assert_close(y.float().cpu().numpy(), ref, f"linear+skipLN {T}x{inn}x{out}")


def test_linear_skip_layernorm_shapes(et, cuda):
    """Widths outside 256..1024 (steps of 128) are refused, not mis-computed."""
    import torch
    x = torch.zeros((16, 64), dtype=torch.float16, device=cuda)
    g = torch.ones((128,), dtype=torch.float16, device=cuda)
    w = torch.zeros((128, 64), dtype=torch.float16, device=cuda)
    with pytest.raises(Exception):
        et.linear_skip_layernorm(x, w, None, None, g, g)
    g = torch.ones((320,), dtype=torch.float16, device=cuda)
    w = torch.zeros((320, 64), dtype=torch.float16, device=cuda)
    with pytest.raises(Exception):
        et.linear_skip_layernorm(x, w, None, None, g, g)
