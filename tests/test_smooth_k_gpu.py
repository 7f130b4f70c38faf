"""k-smoothing on the GPU and the bounded-logit softmax that presumes it.

The reference's callers subtract the per-head mean key before the kernel (``mesh_attention.py:234-237``,
``jax_server.py:276-281``, ``ours_splash_tt.py:136-137``); the wide gate of the bounded-logit softmax is only
safe then.  These tests check the smoothing kernel against the oracle's restatement and that a head whose rows
sit far below the bound comes out as the online softmax would give it, never as silent zeros.
"""
import pytest
import torch

import dtb200
from dtb200 import ops
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def _keys(B, H, S, seed=0, offset=0.0):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, H, S, 128, generator=g)
    k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6) + offset
    return k.to(torch.bfloat16)


@pytest.mark.parametrize("B,H,S,kv_len,offset", [
    (1, 2, 256, None, 0.0),
    (2, 3, 1280, [1243, 1000], 0.5),
    (2, 4, 4608, [4400, 4608], 0.0),
    (1, 2, 20000, [19990], 2.0),          # more than one row chunk per head
    (2, 2, 300, [0, 1], 0.0),             # an empty and a single-row batch element
])
def test_smooth_k_matches_oracle(B, H, S, kv_len, offset):
    k = _keys(B, H, S, seed=S, offset=offset)
    got, norms = dtb200.smooth_k(k.to(DEV), kv_len=kv_len, want_norms=True)
    want = O.smooth_keys(k, kv_len)
    got = got.cpu()
    # The f32 column sums are accumulated in another order than torch's, so a mean may round to the neighbouring
    # bf16 value; its effect on an output is at most one bf16 step of that output.
    diff = (got.float() - want.float()).abs()
    step = want.float().abs().clamp(min=2.0 ** -6) * 2.0 ** -7
    assert (diff <= step).all(), diff.max().item()
    assert (diff > 0).float().mean().item() < 0.02
    if kv_len is not None:
        for b, n in enumerate(kv_len):
            assert got[b, :, n:].abs().max().item() == 0.0 if n < S else True
    want_norms = got.float().norm(dim=-1).amax(dim=(0, 2))
    assert torch.allclose(norms.cpu(), want_norms, rtol=1e-5, atol=1e-6)


def test_smooth_k_in_place_and_strided():
    k = _keys(2, 4, 1024, seed=5, offset=0.25)
    base = k.transpose(1, 2).contiguous().to(DEV)          # stored [B, S, H, D]
    view = base.transpose(1, 2)                            # addressed as [B, H, S, D]
    want = dtb200.smooth_k(view.contiguous(), kv_len=[1000, 1024])
    dtb200.smooth_k(view, kv_len=[1000, 1024], out=view)
    assert torch.equal(view, want)


def _far_below_bound_case():
    """One head whose keys share a large common component u: q rows of norm ~100, one of them pointing along -u.

    The Cauchy-Schwarz bound of the raw keys is ~150 (log2 units) while that row's logits all sit near -130, so a
    constant offset of ceil(150) - 88 would flush every probability of the row to zero.
    """
    g = torch.Generator().manual_seed(11)
    S = 512
    u = torch.randn(128, generator=g)
    u = u / u.norm()
    k = 10.0 * u + 0.5 * torch.randn(1, 1, S, 128, generator=g)
    q = torch.randn(1, 1, S, 128, generator=g)
    q = q / q.norm(dim=-1, keepdim=True) * 100.0
    q[0, 0, 7] = -102.0 * u
    v = torch.randn(1, 1, S, 128, generator=g)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def test_bounded_logit_rows_far_below_the_bound_are_not_flushed():
    q, k, v = _far_below_bound_case()
    ref = O.attention_fp32(q, k, v)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    raw_bound = float(ops.fixed_m_operands(qd, kd)[0, 0])
    assert 106.5 < raw_bound <= 213.0                       # passes the wide gate, fails the halved one
    # un-smoothed keys: the operand is derived with the halved gate, the head stays on the online softmax
    out_raw = dtb200.attention(qd, kd, vd, use_fixed_m=True)
    # the SDPA entry smooths the keys first, as the reference's callers do, and may then use the wide gate
    out_sdpa = dtb200.sdpa(qd, kd, vd, use_fixed_m=True)
    for out in (out_raw, out_sdpa):
        dtb200.check_device_status(DEV)
        err = (out.float().cpu() - ref).abs()
        assert out[0, 0, 7].abs().max().item() > 0.0        # the row along -u is a real average of v, not zeros
        # query rows of norm 100 make the softmax pick single value rows, so outputs reach magnitudes of 2-4 where
        # bf16 steps are 0.016-0.03: the max-abs bound is doubled for this stress case, the mean bound is not
        assert err.max().item() <= 2 * MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL, (err.max().item(), err.mean().item())
    # smoothed keys make every row's largest logit non-negative: the property the wide gate rests on
    ks = dtb200.smooth_k(kd)
    logits = torch.einsum("bhqd,bhkd->bhqk", qd.float(), ks.float())
    assert logits.amax(dim=-1).min().item() >= -1e-2 * logits.abs().max().item()
    mk = ops.fixed_m_operands(qd, ks)
    assert float(mk[1, 0]) == 1.0 and float(mk[0, 0]) < raw_bound


def test_prepass_with_smoothing_feeds_the_wide_gate():
    g = torch.Generator().manual_seed(3)
    B, S, H = 2, 640, 3
    q, k, v = (torch.randn(B, S, H, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    k = (k.float() + 0.75).to(torch.bfloat16)
    kv_len = torch.tensor([600, 640], dtype=torch.int32)
    qo, ko, vo, mk = dtb200.qk_prepass(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len.to(DEV), want_mk=True,
                                       smooth_k=True)
    q0, k0, v0, _ = dtb200.qk_prepass(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len.to(DEV))
    want_k = dtb200.smooth_k(k0, kv_len=kv_len.to(DEV))
    assert torch.equal(ko, want_k) and torch.equal(qo, q0) and torch.equal(vo, v0)
    want_mk = ops.fixed_m_operands(qo, ko, gate=213.0)
    assert torch.equal(mk, want_mk)
    out = dtb200.attention(qo, ko, vo, kv_len=kv_len.to(DEV), use_fixed_m=True, mk=mk)
    ref = O.attention_fp32(q0.cpu(), k0.cpu(), v0.cpu(), kv_len=kv_len)     # smoothing leaves the softmax unchanged
    dtb200.check_device_status(DEV)
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL
