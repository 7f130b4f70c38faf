"""Parity of the fused q/k RMSNorm + rotary + pad-zeroing + layout pre-pass against the CPU oracle."""
import pytest
import torch

import dtb200
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(B, S, H, rotary, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, S, H, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    wq = 1.0 + 0.1 * torch.randn(128, generator=g)
    wk = 1.0 + 0.1 * torch.randn(128, generator=g)
    pos = torch.arange(S, dtype=torch.float32)[:, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, rotary // 2, dtype=torch.float32) / (rotary // 2)))
    ang = pos * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    return q, k, v, wq, wk, cos, sin


def _ulp_close(got, want):
    """Within bf16 rounding of the oracle.  A rotated channel mixes two normalised values of size O(1), each of
    which may round the other way (approximate rsqrt on the GPU), so the bound is two ulps of a value near 1 plus
    two ulps of the result."""
    got, want = got.float().cpu(), want.float()
    tol = want.abs() * 2.0 ** -6 + 2.0 ** -7
    assert ((got - want).abs() <= tol).all(), (got - want).abs().max()


@pytest.mark.parametrize("B,S,H,rotary,kv_len", [
    (2, 300, 4, 96, [300, 250]),      # the H3 layout: 96 of 128 channels rotate, CFG pair with padding
    (1, 129, 3, 128, None),           # all channels rotate
    (1, 64, 2, 0, None),              # no rotary embedding
    (2, 40, 1, 64, [0, 40]),          # a sample that is all padding
])
def test_prepass_matches_oracle(B, S, H, rotary, kv_len):
    q, k, v, wq, wk, cos, sin = _inputs(B, S, H, max(rotary, 16), seed=S)
    rope = (cos, sin) if rotary else None
    want = O.qk_prepass(q, k, v, q_weight=wq, k_weight=wk, eps=1e-5, rope=rope, kv_len=kv_len)
    got = dtb200.qk_prepass(q.to(DEV), k.to(DEV), v.to(DEV), q_weight=wq, k_weight=wk, eps=1e-5, rope=rope, kv_len=kv_len)
    for g, w in zip(got[:3], want):
        assert g.shape == (B, H, S, 128) and g.is_contiguous()
        _ulp_close(g, w)
    assert torch.equal(got[2].cpu(), want[2])          # v only changes layout and gets its padding zeroed
    assert got[3] is None


def test_prepass_takes_strided_projections_and_feeds_attention():
    B, S, H = 2, 640, 4
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, S, 3 * H * 128, generator=g).to(torch.bfloat16).to(DEV)   # one fused projection output
    q, k, v = (t.unflatten(-1, (H, 128)) for t in qkv.chunk(3, dim=-1))            # strided views, no copies
    assert not q.is_contiguous()
    _, _, _, wq, wk, cos, sin = _inputs(B, S, H, 96, seed=6)
    kv_len = [640, 500]
    qn, kn, vn, mk = dtb200.qk_prepass(q, k, v, q_weight=wq, k_weight=wk, rope=(cos, sin), kv_len=kv_len, want_mk=True)
    want = O.qk_prepass(q.cpu(), k.cpu(), v.cpu(), q_weight=wq, k_weight=wk, rope=(cos, sin), kv_len=kv_len)
    for got_t, want_t in zip((qn, kn, vn), want):
        _ulp_close(got_t, want_t)
    # the operand that came for free equals the one a separate pass over the outputs computes
    assert torch.equal(mk, dtb200.fixed_m_operands(qn, kn))
    assert mk[1].tolist() == [1.0] * H
    out = dtb200.attention(qn, kn, vn, kv_len=kv_len, use_fixed_m=True, mk=mk)
    dtb200.check_device_status(DEV)
    ref = O.attention_fp32(qn.cpu(), kn.cpu(), vn.cpu(), kv_len=kv_len)
    err = (out.float().cpu() - ref).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3


def test_prepass_rejects_what_it_cannot_do():
    x = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(NotImplementedError):
        dtb200.qk_prepass(x, x)
    y = torch.zeros(1, 8, 2, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(NotImplementedError):      # rotary width must be a multiple of 16
        dtb200.qk_prepass(y, y, rope=(torch.zeros(8, 24), torch.zeros(8, 24)))
    with pytest.raises(ValueError):
        dtb200.qk_prepass(y, y, rope=(torch.zeros(7, 16), torch.zeros(7, 16)))
