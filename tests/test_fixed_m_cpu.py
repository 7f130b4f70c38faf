"""CPU checks of the host-side fixed-m derivation against the oracle's restatement and the rules the reference
documents for it."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dtb200 import fixed_m as F
from oracle import attn_oracle as O


def _qk(B=2, H=3, S=200, seed=0, gain=1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S, 128, generator=g) * gain
    k = torch.randn(B, H, S, 128, generator=g)
    return q.to(torch.bfloat16), k.to(torch.bfloat16)


def test_constants_and_runtime_operand_match_oracle():
    assert F.FIXED_M_RING_SAFE_BOUND == 106.5 and F.FIXED_M_SAFE_BOUND == 213.0 and F.FIXED_M_RECENTER == 88.0
    q, k = _qk()
    qs = O.scale_query(q, None)
    assert torch.equal(F.fixed_m_operands(qs, k, gate=F.FIXED_M_SAFE_BOUND), O.fixed_m_operands(qs, k))
    qn = F.fixed_m_query_norms(q)
    assert torch.allclose(qn, F.max_row_norm_per_head(q) * (128 ** -0.5) * F.LOG2_E)
    # (B, S, H, D) layout gives the same norms
    assert torch.equal(F.max_row_norm_per_head(q.transpose(1, 2), seq_axis=1), F.max_row_norm_per_head(q))
    ring = F.ring_fixed_m_operands(qn, F.max_row_norm_per_head(k))
    assert torch.equal(ring, O.ring_fixed_m_operands(qn, F.max_row_norm_per_head(k)))
    assert ring[0].tolist() == [106.0] * 3
    with pytest.raises(ValueError):
        F.max_row_norm_per_head(q, seq_axis=3)


def test_sampled_max_logit_is_exact_when_every_row_is_visited_and_bounded_by_cauchy_schwarz():
    q, k = _qk(S=130, seed=1, gain=3.0)
    exact = F.sampled_max_abs_logit(q, k, num_samples=0)
    want = ((q.float() * (128 ** -0.5 * F.LOG2_E)).to(torch.bfloat16).float() @ k.float().transpose(-1, -2)).abs().amax(dim=(0, 2, 3))
    assert torch.allclose(exact, want, rtol=1e-6)
    cs = F.fixed_m_query_norms(q) * F.max_row_norm_per_head(k)
    assert torch.all(exact <= cs * 1.01)
    sampled = F.sampled_max_abs_logit(q, k, num_samples=16, rows_per_chunk=5)
    assert torch.all(sampled <= exact + 1e-6)
    # chunking and layout do not change the result (up to f32 summation order inside the matmul)
    assert torch.allclose(sampled, F.sampled_max_abs_logit(q, k, num_samples=16, rows_per_chunk=64), rtol=1e-6)
    assert torch.allclose(sampled, F.sampled_max_abs_logit(q.transpose(1, 2), k.transpose(1, 2), num_samples=16, seq_axis=1), rtol=1e-6)
    with pytest.raises(ValueError):
        F.sampled_max_abs_logit(q, k, seq_axis=0)


def test_sampling_stride_reaches_the_tail():
    # ceil stride: with 130 rows and 16 samples the stride is 9 and row 126 is visited; make it the outlier
    q, k = _qk(B=1, H=1, S=130, seed=2)
    q[0, 0, 126] *= 50
    hit = F.sampled_max_abs_logit(q, k, num_samples=16)
    assert torch.allclose(hit, F.sampled_max_abs_logit(q, k, num_samples=0))


def test_fp8_measurement_uses_the_quantised_operands():
    q, k = _qk(S=64, seed=3, gain=2.0)
    got = F.sampled_max_abs_logit(q, k, num_samples=0, qk_fp8=True)
    qs = (q.float() * (128 ** -0.5 * F.LOG2_E)).to(torch.bfloat16)
    want = (F.quantize_saturating(qs).float() @ F.quantize_saturating(k).float().transpose(-1, -2)).abs().amax(dim=(0, 2, 3))
    assert torch.allclose(got, want, rtol=1e-6)
    assert F.quantize_saturating(torch.tensor([1e6, -1e6])).float().tolist() == [448.0, -448.0]


def test_static_operand_rules():
    qn, kn = np.array([1.5, 5.0, 9.0]), np.array([11.0, 11.0, 11.0])
    op = F.static_fixed_m_operands(qn, kn, margin_log2=4.0)
    assert op.dtype == np.float32 and op.shape == (2, 3)
    assert op[0].tolist() == [106.0] * 3                       # the largest m the gate permits, for every head
    assert op[1].tolist() == [1.0, 1.0, 1.0]                   # ceil(16.5)+4, 55+4 and 99+4 are all <= 106.5
    # margin only gates eligibility
    assert F.static_fixed_m_operands(qn, kn, margin_log2=8.0)[1].tolist() == [1.0, 1.0, 0.0]
    assert F.static_fixed_m_operands(qn, kn, margin_log2=0.0)[1].tolist() == [1.0, 1.0, 1.0]
    # fp8 inflates the Cauchy-Schwarz bound: 99 * 1.1289 = 111.8 > gate
    assert F.static_fixed_m_operands(qn, kn, margin_log2=0.0, qk_fp8=True)[1].tolist() == [1.0, 1.0, 0.0]
    # a measured max logit can only tighten
    assert F.static_fixed_m_operands(qn, kn, margin_log2=8.0, max_logit=np.array([100.0, 10.0, 60.0]))[1].tolist() == [1.0, 1.0, 1.0]
    assert F.static_fixed_m_operands(qn, kn, margin_log2=4.0, gate=213.0)[0].tolist() == [213.0] * 3
    for bad in (dict(qn_max=qn, mk_h=kn[:2], margin_log2=1.0), dict(qn_max=qn[None], mk_h=kn[None], margin_log2=1.0),
                dict(qn_max=qn, mk_h=kn, margin_log2=-1.0), dict(qn_max=qn, mk_h=kn, margin_log2=1.0, max_logit=np.array([1.0])),
                dict(qn_max=qn, mk_h=kn, margin_log2=1.0, max_logit=np.array([1.0, np.inf, 2.0])),
                dict(qn_max=qn, mk_h=kn, margin_log2=1.0, max_logit=np.array([1.0, -1.0, 2.0]))):
        with pytest.raises(ValueError):
            F.static_fixed_m_operands(**bad)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k = _qk(B=1, H=2, S=256, seed=4, gain=2.0)
        sl = slice(rank * 128, (rank + 1) * 128)
        got = F.sampled_max_abs_logit(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), num_samples=0, group=dist.group.WORLD)
        want = F.sampled_max_abs_logit(q, k, num_samples=0)
        assert torch.allclose(got, want, rtol=1e-6), (got, want)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_measurement_equals_the_global_one(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
