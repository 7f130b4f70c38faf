"""world_size-2 ``gloo`` tests of the multi-GPU drivers' exchange logic on CPU.

The CUDA kernels are replaced by oracle stand-ins through the drivers' injection points, so what is
tested is the host side: the all-to-all layouts of the Ulysses path, the ring schedule, per-shard key
offsets and the running-state merge."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dtb200 import parallel
from oracle import attn_oracle as O

TOL_MAX, TOL_MEAN = 2e-2, 2e-3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(B, H, S, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S, 128, generator=g)
    k = torch.randn(B, H, S, 128, generator=g)
    v = torch.randn(B, H, S, 128, generator=g)
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True)) * 2.0).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    return q, k, v.to(torch.bfloat16)


def _cpu_attend(q, k, v, kv_len=None, scale=None, use_fixed_m=False):
    return O.attention_fp32(q, k, v, kv_len=kv_len, scale=scale).to(torch.bfloat16)


class _CpuState:
    def __init__(self):
        self.parts = []


def _cpu_fold(state, q, k, v, *, scale=None, kv_len=None, kv_offset=0, q_offset=0, use_fixed_m=False, mk=None):
    B, H, Sq, D = q.shape
    lens = [int(x) for x in kv_len] if kv_len is not None else [10 ** 9] * B
    os_, ms, ls = [], [], []
    for b in range(B):
        n = max(0, min(lens[b] - kv_offset, k.shape[2]))
        if n == 0:
            os_.append(torch.zeros(1, H, Sq, D))
            ms.append(torch.full((1, H, Sq, 1), -float("inf")))
            ls.append(torch.zeros(1, H, Sq, 1))
            continue
        o, m, l = O.attention_restated(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n], scale=scale,
                                       emit_residuals=True)
        os_.append(o), ms.append(m), ls.append(l)
    state.parts.append((torch.cat(os_), torch.cat(ms), torch.cat(ls)))
    return state


def _cpu_finalize(state, *, kv_len=None, q_offset=0, zero_padded_rows=True, out=None):
    merged = O.merge_residuals(state.parts)
    if kv_len is not None and zero_padded_rows:
        rows = torch.arange(merged.shape[2]) + q_offset
        for b in range(merged.shape[0]):
            merged[b, :, rows >= int(kv_len[b])] = 0
    return merged.to(torch.bfloat16)


def _worker(rank, world, port, mode, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, S = 2, 4, 384
        q, k, v = _inputs(B, H, S, seed=5)
        kv_len = torch.tensor([S, 301], dtype=torch.int32)
        Sl = S // world
        sl = slice(rank * Sl, (rank + 1) * Sl)
        qs, ks, vs = q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous()
        if mode == "layout":
            xh = parallel.seq_to_heads(qs)
            Hl = H // world
            assert torch.equal(xh, q[:, rank * Hl:(rank + 1) * Hl])
            assert torch.equal(parallel.heads_to_seq(xh), qs)
            got = None
        elif mode == "ulysses":
            got = parallel.ulysses_attention(qs, ks, vs, kv_len=kv_len, attend=_cpu_attend)
        else:
            got = parallel.ring_attention(qs, ks, vs, kv_len=kv_len, new_state=_CpuState, fold=_cpu_fold,
                                          finalize=_cpu_finalize)
        if got is not None:
            ref = O.attention_fp32(q, k, v, kv_len=kv_len)[:, :, sl]
            err = (got.float() - ref).abs()
            assert err.max() <= TOL_MAX and err.mean() <= TOL_MEAN, (err.max(), err.mean())
            for b in range(B):
                pad_from = max(int(kv_len[b]) - rank * Sl, 0)
                assert got[b, :, pad_from:].abs().max() == 0 if pad_from < Sl else True
        open(os.path.join(result_dir, f"ok_{mode}_{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["layout", "ulysses", "ring"])
def test_two_rank_gloo(mode, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok_{mode}_0", f"ok_{mode}_1"]


def test_placement_and_schedule():
    assert parallel.placement(2, 24, 1) == (1, 1)
    assert parallel.placement(2, 24, 2) == (2, 1)       # CFG halves on chip halves, all heads each
    assert parallel.placement(2, 24, 8) == (2, 4)       # two halves x 4 head groups of 6 heads
    assert parallel.placement(1, 40, 8) == (1, 8)
    with pytest.raises(ValueError):
        parallel.placement(1, 24, 16 + 1)
    assert parallel.cfg_subgroups(8, 2) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    for world in (2, 4, 8):
        for rank in range(world):
            sched = parallel.ring_schedule(rank, world)
            assert sched[0] == rank and sorted(sched) == list(range(world))
    # what rank r holds at step t is what rank r-1 held at step t-1
    assert parallel.ring_schedule(3, 8)[2] == parallel.ring_schedule(2, 8)[1]


def _absent_peer_worker(rank, world, port, result_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    q, _, _ = _inputs(1, 2, 64, seed=1)
    if rank == 1:
        # this rank leaves between steps, before the exchange: nothing of its is in flight
        open(os.path.join(result_dir, "left_1"), "w").close()
        os._exit(0)
    try:
        parallel.seq_to_heads(q[:, :, :32].contiguous())
        outcome = "completed"
    except Exception as e:  # the exchange must end with an error, not hang
        outcome = "error:" + type(e).__name__
    open(os.path.join(result_dir, "rank0_" + outcome.split(":")[0]), "w").close()
    os._exit(0)


def test_exchange_with_an_absent_peer_errors_instead_of_hanging(tmp_path):
    """Host-side failure detection: a rank that leaves before a collective makes its peer's call fail within the
    process-group timeout.  CPU ranks only; no GPU work is involved."""
    import time

    t0 = time.time()
    ctx = mp.spawn(_absent_peer_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=False)
    deadline = t0 + 90
    while not ctx.join(timeout=1):
        assert time.time() < deadline, "ranks did not finish: the exchange hung"
    names = sorted(os.listdir(tmp_path))
    assert "left_1" in names and "rank0_error" in names, names
