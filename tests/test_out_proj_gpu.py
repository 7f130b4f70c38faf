"""The output projection behind head-sharded attention output (`dtb_out_proj`) against the CPU oracle.

Tolerance: the kernel multiplies bf16 operands with f32 accumulation; against the oracle's f32 product of the same
bf16 values the f32 partial sums agree to 1e-3 relative to the row scale, and the bf16 output to one bf16 step.
"""
import pytest
import torch

import dtb200
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(B, H, S, N, seed):
    g = torch.Generator().manual_seed(seed)
    o = torch.randn(B, H, S, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(H * 128, N, generator=g) * (H * 128) ** -0.5).to(torch.bfloat16)
    return o, w


@pytest.mark.parametrize("B,H,S,N", [(1, 1, 128, 128), (2, 3, 300, 384), (1, 6, 1000, 3072), (2, 2, 129, 200), (1, 24, 512, 256)])
def test_out_proj_matches_oracle(B, H, S, N):
    o, w = _case(B, H, S, N, seed=S + N)
    got = dtb200.out_proj(o.to(DEV), w.to(DEV))
    dtb200.check_device_status(DEV)
    ref = O.out_proj(o, w)
    assert got.shape == (B, S, N) and got.dtype == torch.bfloat16
    err = (got.float().cpu() - ref).abs()
    assert err.max().item() <= 2.0 ** -7 * max(1.0, ref.abs().max().item()), err.max().item()
    assert err.mean().item() <= 2e-3


def test_out_proj_reads_the_attention_output_in_place():
    """[B, S, H, D] storage viewed as [B, H, S, D], and a weight that is a row slice of the full projection."""
    o, w_full = _case(2, 4, 256, 512, seed=9)
    base = o.transpose(1, 2).contiguous().to(DEV)          # stored [B, S, H, D]
    view = base.transpose(1, 2)
    wd = w_full.to(DEV)
    full = dtb200.out_proj(view, wd)
    assert torch.equal(full, dtb200.out_proj(view.contiguous(), wd))
    # two head shards: partial sums add up to the full projection (what the all-reduce over head shards forms)
    parts = [dtb200.out_proj(view[:, 2 * r:2 * r + 2], wd[256 * r:256 * (r + 1)]).float() for r in range(2)]
    dtb200.check_device_status(DEV)
    err = (parts[0] + parts[1] - O.out_proj(o, w_full).to(DEV)).abs()
    assert err.max().item() <= 3e-2


def test_out_proj_reduce_scatter_with_local_buffers_as_peers():
    """One GPU stands in for four ranks: every rank's heads contribute to all four row shards, which are ordinary
    local f32 buffers here (on a multi-GPU box they are the peers' buffers in symmetric memory)."""
    P, B, H, S, N = 4, 2, 8, 320, 384
    o, w = _case(B, H, S, N, seed=21)
    od, wd = o.to(DEV), w.to(DEV)
    rows = B * S // P
    shards = [torch.zeros(rows, N, dtype=torch.float32, device=DEV) for _ in range(P)]
    Hl = H // P
    for rank in range(P):
        dtb200.out_proj_reduce_(od[:, rank * Hl:(rank + 1) * Hl], wd[rank * Hl * 128:(rank + 1) * Hl * 128],
                                [t.data_ptr() for t in shards], rows)
    dtb200.check_device_status(DEV)
    got = torch.cat(shards).view(B, S, N).cpu()
    ref = O.out_proj(o, w)
    err = (got - ref).abs()
    assert err.max().item() <= 1e-3 * max(1.0, ref.abs().max().item()), err.max().item()


def test_out_proj_partial_rows_and_their_sum_with_local_buffers_as_peers():
    """The default form of the fused reduce-scatter on one GPU: every rank stores bf16 partial rows into its slot of
    each owner's staging buffer, and each owner sums its slots."""
    P, B, H, S, N = 4, 2, 8, 320, 384
    o, w = _case(B, H, S, N, seed=22)
    od, wd = o.to(DEV), w.to(DEV)
    rows = B * S // P
    staged = [torch.full((P, rows, N), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(P)]
    Hl = H // P
    for rank in range(P):
        dtb200.out_proj_reduce_(od[:, rank * Hl:(rank + 1) * Hl], wd[rank * Hl * 128:(rank + 1) * Hl * 128],
                                [t.data_ptr() for t in staged], rows, partials_from=rank)
    got = torch.cat([dtb200.sum_partials(t) for t in staged]).view(B, S, N).float().cpu()
    dtb200.check_device_status(DEV)
    assert not torch.isnan(got).any()
    ref = O.out_proj(o, w)
    err = (got - ref).abs()
    assert err.max().item() <= (P + 1) * 2.0 ** -8 * max(1.0, ref.abs().max().item()), err.max().item()
    # slot r of an owner holds exactly rank r's partial projection of the owner's rows
    part0 = dtb200.out_proj(od[:, :Hl], wd[:Hl * 128]).view(B * S, N)
    assert torch.equal(staged[1][0], part0[rows:2 * rows])


def test_out_proj_rejects_what_it_cannot_do():
    o, w = _case(1, 2, 128, 128, seed=1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        dtb200.out_proj(o, w)
    with pytest.raises(ValueError):
        dtb200.out_proj(o.to(DEV), w[:128].to(DEV))                    # rows of the weight do not match the heads
    with pytest.raises(NotImplementedError):
        dtb200.out_proj(o.float().to(DEV), w.to(DEV))
