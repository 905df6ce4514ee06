"""GPU parity of the fused attention kernel against the oracle: sequence lengths from the
reference's sweep (test/Attention/test_seqlen.cu: 16..512), all mask kinds, fused-QKV layout,
pruned Q/K head width (48), ragged lengths, batch > 1."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _qkv(et, seed, batch, seq, nhead, dh_qk, dh_v, std=1.0):
    T = batch * seq
    q = et.synth.normal(seed, 1, (T, nhead * dh_qk), std)
    k = et.synth.normal(seed, 2, (T, nhead * dh_qk), std)
    v = et.synth.normal(seed, 3, (T, nhead * dh_v), std)
    return q, k, v


@pytest.mark.parametrize("batch,seq,nhead,dh_qk,dh_v", [
    (1, 128, 1, 64, 64), (2, 128, 12, 64, 64), (1, 16, 2, 16, 16), (3, 48, 2, 32, 64),
    (2, 256, 4, 64, 64), (1, 384, 2, 64, 64), (1, 512, 3, 64, 64), (2, 200, 2, 48, 64),
    (1, 1000, 1, 64, 64), (1, 128, 2, 128, 128), (1, 300, 1, 96, 112),
])
@pytest.mark.parametrize("mask_kind", [0, 1])
def test_attention(et, orc, cuda, batch, seq, nhead, dh_qk, dh_v, mask_kind):
    q, k, v = _qkv(et, 100 + seq, batch, seq, nhead, dh_qk, dh_v)
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh_qk, dh_v,
                     mask_kind)
    assert et.device_error() == 0
    ref = orc.attention(q, k, v, batch, seq, nhead, dh_qk, dh_v, mask_kind)
    assert_close(z.float().cpu().numpy(), ref, f"attention b{batch} s{seq} h{nhead} m{mask_kind}",
                 dump=f"attn_{batch}_{seq}_{nhead}_{dh_qk}_{dh_v}_{mask_kind}")


def test_attention_uniform_scores_return_mean_of_v(et, cuda):
    """Constant Q and K give uniform probabilities: Z = mean of V rows (closed form implied
    by the reference's constant-input drivers)."""
    import torch
    batch, seq, nhead, dh = 1, 128, 2, 64
    q = torch.full((seq, nhead * dh), 0.25, dtype=torch.float16, device=cuda)
    v = _dev(et.synth.normal(9, 1, (seq, nhead * dh), 1.0), cuda)
    z = et.attention(q, q, v, batch, seq, nhead, dh, dh)
    ref = v.float().mean(dim=0, keepdim=True).expand(seq, -1)
    assert torch.allclose(z.float(), ref, atol=3e-3)


def test_attention_fused_qkv_layout(et, orc, cuda):
    """Q, K, V as column ranges of one [T, 2*kdim + vdim] buffer (Attention.h:258-263)."""
    batch, seq, nhead, dh = 2, 128, 4, 64
    kdim = vdim = nhead * dh
    buf = et.synth.normal(77, 1, (batch * seq, 2 * kdim + vdim), 1.0)
    d = _dev(buf, cuda)
    z = et.attention(d[:, :kdim], d[:, kdim:2 * kdim], d[:, 2 * kdim:], batch, seq, nhead, dh, dh)
    assert et.device_error() == 0
    ref = orc.attention(buf[:, :kdim], buf[:, kdim:2 * kdim], buf[:, 2 * kdim:], batch, seq, nhead,
                        dh, dh)
    assert_close(z.float().cpu().numpy(), ref, "fused qkv layout")


@pytest.mark.parametrize("seq", [128, 384])
def test_attention_padding_mask(et, orc, cuda, seq):
    batch, nhead, dh = 4, 2, 64
    q, k, v = _qkv(et, 55, batch, seq, nhead, dh, dh)
    vl = np.array([seq, seq // 3, 1, 130 if seq > 130 else 17], dtype=np.int32)
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh, dh, 2,
                     None, _dev(vl, cuda))
    assert et.device_error() == 0
    ref = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 2, None, vl)
    assert_close(z.float().cpu().numpy(), ref, "padding mask")


def test_attention_zero_valid_length_gives_zeros(et, cuda):
    import torch
    batch, seq, nhead, dh = 2, 64, 1, 32
    q = _dev(et.synth.normal(3, 1, (batch * seq, dh), 1.0), cuda)
    vl = _dev(np.array([0, seq], dtype=np.int32), cuda)
    z = et.attention(q, q, q, batch, seq, nhead, dh, dh, 2, None, vl)
    assert et.device_error() == 0
    assert torch.all(z[:seq] == 0)
    assert torch.isfinite(z.float()).all()


@pytest.mark.parametrize("seq", [64, 128, 272])
def test_attention_additive_mask(et, orc, cuda, seq):
    """General additive [seq, seq] mask; the causal one of Attention.h:97-104 must agree with
    ET_MASK_CAUSAL."""
    batch, nhead, dh = 2, 2, 64
    q, k, v = _qkv(et, 66, batch, seq, nhead, dh, dh)
    causal = np.where(np.tril(np.ones((seq, seq), bool)), 0.0, -np.inf).astype(np.float16)
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh, dh, 3,
                     _dev(causal, cuda))
    assert et.device_error() == 0
    ref = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 1)
    assert_close(z.float().cpu().numpy(), ref, "additive causal")
    soft = et.synth.normal(67, 9, (seq, seq), 1.0)
    soft[3, :] = -np.inf  # one fully dropped query row -> zeros
    z = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), batch, seq, nhead, dh, dh, 3,
                     _dev(soft, cuda))
    ref = orc.attention(q, k, v, batch, seq, nhead, dh, dh, 3, soft.astype(np.float32))
    assert_close(z.float().cpu().numpy(), ref, "additive soft")


def test_attention_is_deterministic(et, cuda):
    import torch
    q, k, v = _qkv(et, 88, 2, 256, 4, 64, 64)
    a = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), 2, 256, 4, 64, 64, 1)
    b = et.attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), 2, 256, 4, 64, 64, 1)
    assert torch.equal(a, b)
