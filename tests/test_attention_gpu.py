"""Parity of the CUDA attention path (called through the C ABI) against the CPU oracle on B200.

Tolerance of the path: bf16 output within max-abs 2e-2 and mean-abs 2e-3 of the fp32-softmax oracle
on the same seeded inputs; padded query rows exactly zero.
"""
import os

import numpy as np
import pytest
import torch

import dtb200
from dtb200.inputs import CONFIGS, make_inputs
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu

MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"


def _rand(B, H, Sq, Skv, seed=0, gain=1.0, Hkv=None):
    g = torch.Generator().manual_seed(seed)
    Hkv = H if Hkv is None else Hkv
    q = torch.randn(B, H, Sq, 128, generator=g)
    k = torch.randn(B, Hkv, Skv, 128, generator=g)
    v = torch.randn(B, Hkv, Skv, 128, generator=g)
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6) * gain).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    return q, k, v.to(torch.bfloat16)


def _check(out, ref, kv_len=None, tol_scale=1.0):
    dtb200.check_device_status(DEV)
    out = out.float().cpu()
    assert not torch.isnan(out).any()
    err = (out - ref).abs()
    assert err.max().item() <= MAX_ABS_TOL * tol_scale, err.max().item()
    assert err.mean().item() <= MEAN_ABS_TOL * tol_scale, err.mean().item()
    if kv_len is not None:
        for b, n in enumerate(kv_len):
            assert out[b, :, int(n):].abs().max().item() == 0.0 if int(n) < out.shape[2] else True


@pytest.mark.parametrize("name", ["joint_small", "peaked_cross"])
def test_golden_vectors(name):
    data = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    q, k, v = (torch.from_numpy(data[n]).view(torch.bfloat16) for n in ("q", "k", "v"))
    kv_len = data["kv_len"].tolist()
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len)
    _check(out, torch.from_numpy(data["out_fp32"]), kv_len)


def test_config1_full_call_matches_both_oracles():
    cfg = CONFIGS["c1_image512_cpu"]
    q, k, v, kv_len = make_inputs(cfg, 0)
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len.to(DEV))
    _check(out, O.attention_fp32(q, k, v, kv_len=kv_len), kv_len.tolist())
    n = int(kv_len[0])
    restated = O.attention_restated(q, k, v, kv_len=n, use_fixed_m=True).float()
    err = (out.float().cpu()[:, :, :n] - restated[:, :, :n]).abs()
    assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL


@pytest.mark.parametrize("use_fixed_m", [False, True])
def test_restated_reference_kernel_agrees_on_config2_heads(use_fixed_m):
    """Three heads of one C2 batch element at full length (4608 tokens, 36 key tiles, its own padding) against the
    step-by-step restatement of the reference kernel (bf16 rounding of the scaled query, exp2, bf16 P, the
    reference's 1024/2048 tiling, online or per-head constant offset): the two are different tilings of the same
    arithmetic and must agree within the path's tolerance, as each does with the fp32 oracle."""
    cfg = CONFIGS["c2_image1024"]
    q, k, v, kv_len = make_inputs(cfg, 11, heads=3)
    q, k, v = q[1:2], k[1:2], v[1:2]
    n = int(kv_len[1])
    assert n < cfg.seq
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=[n], use_fixed_m=use_fixed_m)
    dtb200.check_device_status(DEV)
    restated = O.attention_restated(q, k, v, kv_len=n, use_fixed_m=use_fixed_m).float()
    err = (out.float().cpu()[:, :, :n] - restated[:, :, :n]).abs()
    assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL, (err.max().item(), err.mean().item())
    fp32 = O.attention_fp32(q, k, v, kv_len=[n])
    err = (restated[:, :, :n] - fp32[:, :, :n]).abs()
    assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL


@pytest.mark.parametrize("call_index", [0, 7, 59])
def test_config2_sampled_rows(call_index):
    cfg = CONFIGS["c2_image1024"]
    q, k, v, kv_len = make_inputs(cfg, call_index)
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len.to(DEV))
    dtb200.check_device_status(DEV)
    rows = torch.cat([torch.arange(0, cfg.seq, 53), torch.arange(cfg.seq - 320, cfg.seq)]).unique()
    ref = O.attention_fp32(q, k, v, kv_len=kv_len, rows=rows)
    _check(out[:, :, rows.to(DEV)], ref)
    for b in range(cfg.batch):
        assert out[b, :, int(kv_len[b]):].abs().max().item() == 0.0


@pytest.mark.parametrize("B,H,Sq,Skv,kv_len,gain", [
    (1, 1, 256, 256, None, 1.0),
    (1, 2, 300, 300, None, 1.0),          # ragged: not a multiple of the tile
    (1, 1, 130, 70, None, 1.0),           # shorter than one tile on both axes
    (1, 1, 256, 256, [1], 1.0),           # a single valid key
    (3, 1, 384, 384, [127, 128, 129], 1.0),   # around a tile boundary
    (2, 2, 640, 640, [640, 400], 2.0),    # per-sample lengths (a CFG pair)
    (1, 4, 128, 2048, None, 1.0),         # short-query cross attention
    (1, 2, 700, 900, [801], 10.0),        # peaked softmax, ragged, padded
    (2, 1, 512, 512, [0, 512], 1.0),      # one sample with no valid key at all
])
def test_edge_shapes(B, H, Sq, Skv, kv_len, gain):
    q, k, v = _rand(B, H, Sq, Skv, seed=Sq + Skv, gain=gain)
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len)
    _check(out, O.attention_fp32(q, k, v, kv_len=kv_len), kv_len if Sq == Skv else None)


def test_gqa_and_strided_inputs():
    q, k, v = _rand(2, 4, 384, 384, seed=11, Hkv=2)
    ref = O.attention_fp32(q, k, v)
    # [B, S, H, D] storage viewed as [B, H, S, D]: the layout diffusers hands to its attention hook
    qs = q.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    ks = k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    vs = v.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    assert not qs.is_contiguous()
    _check(dtb200.attention(qs, ks, vs), ref)
    out_view = torch.empty(2, 384, 4, 128, dtype=torch.bfloat16, device=DEV).transpose(1, 2)
    dtb200.attention(qs, ks, vs, out=out_view)
    _check(out_view, ref)


def test_padding_content_cannot_reach_real_rows():
    q, k, v = _rand(1, 2, 512, 512, seed=12)
    n = 401
    base = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=n).clone()
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    # finite garbage, as the reference's own pad-fill diagnosis uses (non-finite padded V would
    # poison 0 * v products in any flash kernel, the reference's included; its callers zero padded V)
    q2[:, :, n:] = 3.0
    k2[:, :, n:] = torch.randn_like(k2[:, :, n:]) * 50
    v2[:, :, n:] = 3.0e4
    other = dtb200.attention(q2.to(DEV), k2.to(DEV), v2.to(DEV), kv_len=n)
    dtb200.check_device_status(DEV)
    assert torch.equal(base, other)


def test_padded_call_equals_unpadded_call():
    q, k, v = _rand(1, 2, 640, 640, seed=13)
    n = 517
    a = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=n)[:, :, :n]
    b = dtb200.attention(q[:, :, :n].contiguous().to(DEV), k[:, :, :n].contiguous().to(DEV),
                         v[:, :, :n].contiguous().to(DEV))
    dtb200.check_device_status(DEV)
    assert torch.equal(a, b)


def test_zero_padded_rows_flag_off_keeps_padded_queries():
    q, k, v = _rand(1, 1, 256, 256, seed=14)
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=100, zero_padded_rows=False)
    ref = O.attention_fp32(q, k, v, kv_len=100, zero_padded_rows=False)
    _check(out, ref)
    assert out[:, :, 100:].abs().max().item() > 0


@pytest.mark.parametrize("gain", [1.0, 6.0])
def test_bounded_logit_mode_equals_online(gain):
    q, k, v = _rand(2, 3, 700, 700, seed=15, gain=gain)
    kv_len = [650, 300]
    ref = O.attention_fp32(q, k, v, kv_len=kv_len)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    mk = dtb200.fixed_m_operands(qd, kd)
    want = O.fixed_m_operands((q.float() * (128 ** -0.5) * O.LOG2_E), k)
    assert torch.equal(mk.cpu(), want)
    fixed = dtb200.attention(qd, kd, vd, kv_len=kv_len, use_fixed_m=True)
    _check(fixed, ref, kv_len)
    online = dtb200.attention(qd, kd, vd, kv_len=kv_len)
    assert (fixed.float() - online.float()).abs().max().item() <= 4e-3 * gain


def test_ineligible_heads_fall_back_to_online_softmax():
    q, k, v = _rand(1, 2, 256, 256, seed=16)
    q[:, 1] *= 30                        # head 1 blows the gate, head 0 stays eligible
    mk = dtb200.fixed_m_operands(q.to(DEV), k.to(DEV))
    assert mk[1].tolist() == [1.0, 0.0]
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), use_fixed_m=True, mk=mk)
    _check(out, O.attention_fp32(q, k, v), tol_scale=2.0)


@pytest.mark.parametrize("splits", [0, 2, 3, 7])
def test_split_kv_matches_unsplit(splits):
    q, k, v = _rand(2, 2, 300, 3000, seed=17, gain=3.0)
    kv_len = [2999, 1500]
    out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len, num_splits=splits,
                           zero_padded_rows=False)
    _check(out, O.attention_fp32(q, k, v, kv_len=kv_len, zero_padded_rows=False))


def test_residual_ring_steps_match_single_pass():
    q, k, v = _rand(1, 2, 1024, 1024, seed=18, gain=4.0)
    n = 900
    ref = O.attention_fp32(q, k, v, kv_len=n)
    qd = q.to(DEV)
    state = dtb200.ResidualState(1, 2, 1024, torch.device(DEV))
    for i in (2, 0, 3, 1):               # any order: the merge is order-free
        sl = slice(i * 256, (i + 1) * 256)
        dtb200.residual_attention_(state, qd, k[:, :, sl].contiguous().to(DEV), v[:, :, sl].contiguous().to(DEV),
                                   kv_len=n, kv_offset=i * 256)
    out = dtb200.finalize_residual(state, kv_len=n)
    _check(out, ref, [n])


def test_residual_parts_merge_like_the_reference_ring():
    q, k, v = _rand(1, 2, 384, 768, seed=19, gain=2.0)
    ref = O.attention_fp32(q, k, v)
    qd = q.to(DEV)
    mk = O.ring_fixed_m_operands(O.max_row_norm_per_head(q.float() * (128 ** -0.5) * O.LOG2_E),
                                 O.max_row_norm_per_head(k)).to(DEV)
    for use_fixed_m in (False, True):
        parts = []
        for i in range(3):
            sl = slice(i * 256, (i + 1) * 256)
            o, m, l = dtb200.residual_attention(qd, k[:, :, sl].contiguous().to(DEV), v[:, :, sl].contiguous().to(DEV),
                                                use_fixed_m=use_fixed_m, mk=mk if use_fixed_m else None)
            assert o.shape == (1, 2, 384, 128) and m.shape == (1, 2, 384, 1) and l.shape == (1, 2, 384, 1)
            parts.append((o.cpu(), m.cpu(), l.cpu()))
        dtb200.check_device_status(DEV)
        if use_fixed_m:
            assert torch.all(parts[0][1] == 106.0 - 88.0)
        err = (O.merge_residuals(parts) - ref).abs()
        assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL


def test_sdpa_signature_ignores_unsupported_arguments():
    q, k, v = _rand(1, 2, 256, 256, seed=20)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    a = dtb200.sdpa(qd, kd, vd, attn_mask=torch.ones(1), dropout_p=0.5, is_causal=True, scale=None, enable_gqa=True)
    b = dtb200.attention(qd, kd, vd)
    dtb200.check_device_status(DEV)
    assert torch.equal(a, b)


def test_unsupported_inputs_raise_instead_of_falling_back():
    x = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(NotImplementedError):
        dtb200.attention(x, x, x)
    y = torch.zeros(1, 2, 128, 128, dtype=torch.float16, device=DEV)
    with pytest.raises(NotImplementedError):
        dtb200.attention(y, y, y)
    z = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(NotImplementedError):           # E4M3 scores with the bounded-logit mode need a calibrated operand
        dtb200.attention(z, z, z, qk_fp8=True, use_fixed_m=True)


@pytest.mark.parametrize("B,H,S,kv_len", [(1, 2, 512, None), (2, 3, 1100, [1100, 777])])
def test_qk_fp8_variant_matches_oracle_on_quantised_operands(B, H, S, kv_len):
    from dtb200 import fixed_m as F

    q, k, v = _rand(B, H, S, S, seed=31, gain=1.5)
    qd, kd = q.to(DEV), k.to(DEV)
    c = (128 ** -0.5) * F.LOG2_E
    q8 = dtb200.quantize_e4m3(qd, mult=c)
    k8 = dtb200.quantize_e4m3(kd)
    assert q8.dtype == torch.float8_e4m3fn and q8.shape == q.shape
    # the cast is the saturating round-to-nearest of the reference
    assert torch.equal(q8.float().cpu(), F.quantize_saturating(q.float() * c).float())
    assert torch.equal(k8.float().cpu(), F.quantize_saturating(k).float())
    assert dtb200.quantize_e4m3((qd.float() * 1e4).to(torch.bfloat16)).float().abs().max().item() == 448.0
    out = dtb200.attention(qd, kd, v.to(DEV), kv_len=kv_len, qk_fp8=True)
    # oracle on the same quantised operands: the logits are already in log2 units, so softmax scale = ln 2
    ref = O.attention_fp32(q8.float().cpu(), k8.float().cpu(), v, kv_len=kv_len, scale=1.0 / F.LOG2_E)
    _check(out, ref, kv_len)
    # the variant is lossy by design (E4M3 keeps 3 mantissa bits of q and k): it stays near the full-precision
    # result but is not held to the bf16 path's tolerance
    full = O.attention_fp32(q, k, v, kv_len=kv_len)
    err = (out.float().cpu() - full).abs()
    assert err.max().item() <= 0.25 and err.mean().item() <= 2e-2


def test_residual_ring_with_e4m3_scores_and_the_ring_operand():
    """The reference's fastest ring configuration: E4M3 q/k with the bounded-logit softmax on one operand for all
    steps (``fixed_m_bound.py:121-155, 313-316``).  Four shards folded in ring order, against the oracle on the same
    quantised operands."""
    from dtb200 import fixed_m as F

    B, H, S, n = 2, 3, 1024, [1000, 1024]
    q, k, v = _rand(B, H, S, S, seed=41, gain=1.5)
    c = (128 ** -0.5) * F.LOG2_E
    q8, k8 = dtb200.quantize_e4m3(q.to(DEV), mult=c), dtb200.quantize_e4m3(k.to(DEV))
    qn, kn = dtb200.ops.row_norm_maxima(q.to(DEV), k.to(DEV))
    assert torch.allclose(qn.cpu(), F.fixed_m_query_norms(q), rtol=1e-5) and torch.allclose(kn.cpu(), F.max_row_norm_per_head(k), rtol=1e-5)
    mk = F.ring_fixed_m_operands(qn * (1 + 2.0 ** -4), kn * (1 + 2.0 ** -4))
    assert torch.all(mk[1] == 1.0) and torch.all(mk[0] == 106.0)
    ref = O.attention_fp32(q8.float().cpu(), k8.float().cpu(), v, kv_len=n, scale=1.0 / F.LOG2_E)
    for pre_cast in (False, True):
        state = dtb200.ResidualState(B, H, S, torch.device(DEV))
        for i in (1, 0, 3, 2):
            sl = slice(i * 256, (i + 1) * 256)
            ks = (k8 if pre_cast else k.to(DEV))[:, :, sl].contiguous()
            dtb200.residual_attention_(state, q8 if pre_cast else q.to(DEV), ks, v[:, :, sl].contiguous().to(DEV),
                                       kv_len=n, kv_offset=i * 256, use_fixed_m=True, mk=mk, qk_fp8=True)
        assert torch.all(state.m == 106.0 - 88.0)
        _check(dtb200.finalize_residual(state, kv_len=n), ref, n)
    o, m, l = dtb200.residual_attention(q.to(DEV), k.to(DEV), v.to(DEV), qk_fp8=True)   # online softmax, one shard
    _check(dtb200.finalize_residual(_state_of(o, m, l)), O.attention_fp32(q8.float().cpu(), k8.float().cpu(), v, scale=1.0 / F.LOG2_E))


def _state_of(o, m, l):
    st = dtb200.ResidualState(o.shape[0], o.shape[1], o.shape[2], o.device)
    st.o, st.m, st.l, st.fresh = o, m.squeeze(-1).contiguous(), l.squeeze(-1).contiguous(), False
    return st


def test_full_size_properties_config2():
    """At full size: linearity in V and invariance to k-smoothing, which need no oracle pass."""
    cfg = CONFIGS["c2_image1024"]
    q, k, v, kv_len = make_inputs(cfg, 3, device=DEV)
    base = dtb200.attention(q, k, v, kv_len=kv_len).float()
    doubled = dtb200.attention(q, k, (v.float() * 2).to(torch.bfloat16), kv_len=kv_len).float()
    assert (doubled - 2 * base).abs().max().item() <= 2e-3
    valid = (torch.arange(cfg.seq, device=DEV)[None, :] < kv_len[:, None])[:, None, :, None]
    mean = (k.float() * valid).sum(2, keepdim=True) / kv_len.float()[:, None, None, None]
    smoothed = ((k.float() - mean) * valid).to(torch.bfloat16)
    out_s = dtb200.attention(q, smoothed, v, kv_len=kv_len).float()
    dtb200.check_device_status(DEV)
    err = (out_s - base).abs()
    assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL


def test_randomised_shapes_against_oracle():
    """A seeded sweep over ragged shapes, GQA ratios, per-sample lengths and logit scales; outputs are pre-filled with
    NaN canaries, none of which may survive (every row of the output is written, padded ones as zeros)."""
    g = torch.Generator().manual_seed(2024)
    for case in range(24):
        B = int(torch.randint(1, 4, (1,), generator=g))
        Hkv = int(torch.randint(1, 4, (1,), generator=g))
        H = Hkv * int(torch.randint(1, 3, (1,), generator=g))
        Sq = int(torch.randint(1, 700, (1,), generator=g))
        Skv = Sq if case % 3 else int(torch.randint(1, 900, (1,), generator=g))
        gain = float(torch.rand(1, generator=g)) * 5 + 0.5
        kv_len = None
        if case % 2:
            kv_len = [int(torch.randint(1, Skv + 1, (1,), generator=g)) for _ in range(B)]
        q, k, v = _rand(B, H, Sq, Skv, seed=1000 + case, gain=gain, Hkv=Hkv)
        out = torch.full((B, H, Sq, 128), float("nan"), dtype=torch.bfloat16, device=DEV)
        dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_len=kv_len, out=out,
                         use_fixed_m=bool(case % 4 == 3), num_splits=(0, 1, 2)[case % 3])
        dtb200.check_device_status(DEV)
        assert not torch.isnan(out.float()).any(), f"case {case}: NaN canary survived"
        ref = O.attention_fp32(q, k, v, kv_len=kv_len)
        err = (out.float().cpu() - ref).abs()
        assert err.max().item() <= MAX_ABS_TOL and err.mean().item() <= MEAN_ABS_TOL, (case, B, H, Hkv, Sq, Skv, kv_len, gain)


def test_concurrent_streams_share_nothing_they_should_not():
    """Two streams running unsplit calls at once must not disturb each other (no hidden global scratch)."""
    q, k, v = _rand(2, 4, 1024, 1024, seed=77)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    want = dtb200.attention(qd, kd, vd, num_splits=1).clone()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = []
    for _ in range(4):
        for s in (s1, s2):
            with torch.cuda.stream(s):
                outs.append(dtb200.attention(qd, kd, vd, num_splits=1))
    dtb200.check_device_status(DEV)
    assert all(torch.equal(o, want) for o in outs)


@pytest.mark.parametrize("pattern", ["rising", "late_spike", "mixed_rows"])
def test_offsets_that_move_after_the_first_tile(pattern):
    """The kernel exponentiates the first half of a tile with the offset it already has and only then confirms it
    against the tile's maximum; here the maximum does outgrow the offset (by more than the 2^8 of slack) in later
    tiles - in every tile, in a single late one, or only for some rows of a warp - so the speculated half must be
    thrown away, the accumulator rescaled, and the result still match the oracle."""
    g = torch.Generator().manual_seed(21)
    S = 1024                                              # 8 key tiles
    u = torch.randn(128, generator=g)
    u = u / u.norm()
    noise = 0.05 * torch.randn(1, 2, S, 128, generator=g)
    ramp = torch.zeros(S)
    if pattern == "rising":
        ramp = torch.linspace(0.0, 80.0, S)               # logits climb ~13 log2 units per tile
    elif pattern == "late_spike":
        ramp[700:] = 9.0                                  # one jump inside the sixth tile
    else:
        ramp[520:] = 9.0
    k = ramp[None, None, :, None] * u + noise
    q = torch.randn(1, 2, 512, 128, generator=g) * 0.3
    q = q + 10.0 * u
    if pattern == "mixed_rows":
        q[:, :, ::3] -= 20.0 * u                          # every third row sees the jump as a drop instead
    v = torch.randn(1, 2, S, 128, generator=g)
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    ref = O.attention_fp32(q, k, v)
    for splits in (1, 2):
        out = dtb200.attention(q.to(DEV), k.to(DEV), v.to(DEV), num_splits=splits)
        _check(out, ref)
