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
