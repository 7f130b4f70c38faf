"""CPU checks of the oracle: its two formulations against each other, against the committed golden
vectors, and against the invariants the reference documents for its kernel."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import attn_oracle as O

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")

# Parity tolerance of the path: bf16 output against the fp32-softmax reference.
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def _rand(B, H, Sq, Skv, seed=0, gain=1.0, Hkv=None):
    g = torch.Generator().manual_seed(seed)
    Hkv = H if Hkv is None else Hkv
    q = torch.randn(B, H, Sq, 128, generator=g)
    k = torch.randn(B, Hkv, Skv, 128, generator=g)
    v = torch.randn(B, Hkv, Skv, 128, generator=g)
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6) * gain).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    return q, k, v.to(torch.bfloat16)


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_golden_vectors_reproduce(name):
    data = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    q, k, v, kv_len = make_golden.make_case(name)
    assert np.array_equal(q.view(torch.int16).numpy(), data["q"])
    assert np.array_equal(k.view(torch.int16).numpy(), data["k"])
    assert np.array_equal(v.view(torch.int16).numpy(), data["v"])
    ref = O.attention_fp32(q, k, v, kv_len=kv_len).numpy()
    np.testing.assert_allclose(ref, data["out_fp32"], rtol=0, atol=2e-6)


@pytest.mark.parametrize("use_fixed_m", [False, True])
@pytest.mark.parametrize("blocks", [(1024, 2048, 1024), (128, 256, 128), (96, 160, 160)])
def test_restated_reference_matches_fp32(use_fixed_m, blocks):
    q, k, v = _rand(1, 2, 300, 420, seed=1, gain=1.5)
    ref = O.attention_fp32(q, k, v, kv_len=401)
    got = O.attention_restated(q, k, v, kv_len=401, block_q=blocks[0], block_kv=blocks[1],
                               block_kv_compute=blocks[2], use_fixed_m=use_fixed_m).float()
    d = (got[:, :, :401] - ref[:, :, :401]).abs()
    assert d.max() <= MAX_ABS_TOL and d.mean() <= MEAN_ABS_TOL


def test_padded_call_equals_unpadded():
    # A padded call with kv_len attends exactly like the unpadded one (splash.py:204-207), whatever
    # the padded keys and values hold.
    q, k, v = _rand(1, 2, 200, 256, seed=2)
    n = 173
    base = O.attention_fp32(q[:, :, :n], k[:, :, :n], v[:, :, :n])
    k2, v2 = k.clone(), v.clone()
    k2[:, :, n:] = 1e3
    v2[:, :, n:] = -7.0
    padded = O.attention_fp32(q, k2, v2, kv_len=n)
    assert torch.equal(padded[:, :, :n], base)
    assert padded[:, :, n:].abs().max() == 0


def test_k_smoothing_invariance():
    # softmax is invariant to subtracting the per-head key mean (mesh_attention.py:234-237)
    q, k, v = _rand(1, 2, 128, 192, seed=3, gain=2.0)
    a = O.attention_fp32(q, k.float(), v)
    b = O.attention_fp32(q, O.smooth_keys(k.float()), v)
    assert (a - b).abs().max() < 1e-5


def test_fixed_m_operand_and_gate():
    q, k, _ = _rand(2, 3, 64, 80, seed=4)
    mk = O.fixed_m_operands(O.scale_query(q, None), k)
    assert mk.shape == (2, 3)
    # unit-weight qk-norm: |q*scale*log2e| ~ 1.4427, |k| ~ sqrt(128)  ->  bound ~ 16.3
    assert torch.all(mk[0] == 17) and torch.all(mk[1] == 1)
    big = O.fixed_m_operands(O.scale_query(q * 20, None), k)
    assert torch.all(big[1] == 0)
    ring = O.ring_fixed_m_operands(torch.tensor([1.5, 20.0]), torch.tensor([11.3, 11.3]))
    assert ring[0].tolist() == [106.0, 106.0] and ring[1].tolist() == [1.0, 0.0]


@pytest.mark.parametrize("use_fixed_m", [False, True])
def test_ring_merge_matches_single_pass(use_fixed_m):
    q, k, v = _rand(1, 2, 96, 512, seed=5, gain=4.0)
    ref = O.attention_fp32(q, k, v)
    mk = None
    if use_fixed_m:
        qn = O.max_row_norm_per_head(O.scale_query(q, None))
        mk = O.ring_fixed_m_operands(qn, O.max_row_norm_per_head(k))
    parts = [O.attention_restated(q, k[:, :, i:i + 128], v[:, :, i:i + 128], emit_residuals=True,
                                  use_fixed_m=use_fixed_m, mk=mk) for i in range(0, 512, 128)]
    merged = O.merge_residuals(parts)
    d = (merged - ref).abs()
    assert d.max() <= MAX_ABS_TOL and d.mean() <= MEAN_ABS_TOL


def test_merge_ignores_empty_shards():
    q, k, v = _rand(1, 1, 32, 128, seed=6)
    full = O.attention_restated(q, k, v, emit_residuals=True)
    empty = (torch.zeros_like(full[0]), torch.full_like(full[1], -float("inf")), torch.zeros_like(full[2]))
    merged = O.merge_residuals([full, empty])
    ref = full[0] / full[2]
    assert torch.allclose(merged, ref, atol=1e-6)


def test_gqa_maps_query_heads_to_kv_heads():
    q, k, v = _rand(1, 4, 64, 64, seed=7, Hkv=2)
    got = O.attention_fp32(q, k, v)
    want = O.attention_fp32(q, k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1))
    assert torch.equal(got, want)


def test_sampled_rows_match_full():
    q, k, v = _rand(1, 1, 200, 200, seed=8)
    rows = torch.arange(0, 200, 7)
    full = O.attention_fp32(q, k, v, kv_len=150)
    part = O.attention_fp32(q, k, v, kv_len=150, rows=rows)
    assert torch.equal(part, full[:, :, rows])


def test_prepass_oracle_properties():
    # RMSNorm makes every kept row's mean square ~1 (unit weights), the rotation preserves each rotated pair's norm,
    # channels past `rotary` pass through, padded rows are zero and the layout is (B, H, S, D).
    g = torch.Generator().manual_seed(9)
    q = torch.randn(2, 50, 3, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(2, 50, 3, 128, generator=g).to(torch.bfloat16)
    ang = torch.arange(50, dtype=torch.float32)[:, None] * torch.linspace(0.01, 1.0, 48)[None, :]
    cos, sin = torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1)
    qn, kn, vn = O.qk_prepass(q, k, None, rope=(cos, sin), kv_len=[50, 31])
    assert vn is None and qn.shape == (2, 3, 50, 128)
    plain_q, _, _ = O.qk_prepass(q, k, None)
    assert torch.allclose(plain_q.float().pow(2).mean(-1), torch.ones(2, 3, 50), atol=2e-2)
    assert torch.equal(qn[0, :, :, 96:], plain_q[0, :, :, 96:])
    pair = lambda t: t[..., :48].float().pow(2) + t[..., 48:96].float().pow(2)
    assert torch.allclose(pair(qn[0]), pair(plain_q[0]), rtol=3e-2, atol=1e-3)
    assert qn[1, :, 31:].abs().max() == 0 and kn[1, :, 31:].abs().max() == 0 and qn[1, :, :31].abs().max() > 0
