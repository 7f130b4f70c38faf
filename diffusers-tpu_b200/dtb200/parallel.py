"""Single-box multi-GPU placements of the joint attention: one process per GPU, NCCL over NVLink.

Three placements, as in the reference:

* **resident head-parallel shards** with CFG halves on chip halves — every rank already holds
  ``[B_local, H_local, S, D]`` and runs the local kernel; no collective
  (``diffusers_tpu/kernels/mesh_attention.py:72-145``: heads over devices, batch on the first mesh axis).
* **Ulysses** — the stream is sequence-sharded ``[B, H, S/P, D]``; an all-to-all turns it into head
  shards ``[B, H/P, S, D]`` for q, k and v, the local kernel runs, and the inverse all-to-all returns
  the output to sequence shards (``diffusers_tpu/backends/qwen21_core_tt.py:61-66, 108-129``,
  ``diffusers_tpu/models/qwen_image_21/jax_dit.py:244-285``).
* **ring-KV** — q stays put, the K/V shards rotate ``P - 1`` times and every step is folded into a running
  ``(o, m, l)`` by the residual kernel; the merge is the m-invariant LSE-space one that
  ``diffusers_tpu/kernels/splash.py:657-662, 688-691`` prescribes.  The reference ships the device-local
  kernel only; this driver is built from that prose.

The compute callables default to the CUDA kernels; tests inject CPU stand-ins to exercise the exchange
logic on ``gloo`` ranks.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def placement(batch: int, heads: int, world: int) -> Tuple[int, int]:
    """``(batch_groups, head_groups)``: batch elements (the CFG pair) are dealt out first, then heads."""
    bg = min(batch, world)
    while world % bg or batch % bg:
        bg -= 1
    hg = world // bg
    if heads % hg:
        raise ValueError(f"{heads} heads do not divide over {hg} ranks per batch group")
    return bg, hg


def cfg_subgroups(world: int, batch_groups: int) -> List[List[int]]:
    """Rank lists of the chip halves (or quarters): consecutive ranks share a batch element."""
    per = world // batch_groups
    return [list(range(g * per, (g + 1) * per)) for g in range(batch_groups)]


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def seq_to_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    """``[B, H, S/P, D]`` (all heads of one sequence shard) -> ``[B, H/P, S, D]`` (whole sequence of one head shard)."""
    P = _world(group)
    if P == 1:
        return x
    B, H, Sl, D = x.shape
    if H % P:
        raise ValueError(f"{H} heads do not divide over {P} ranks")
    Hl = H // P
    send = x.reshape(B, P, Hl, Sl, D).permute(1, 0, 2, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[r] is rank r's sequence shard of my heads
    return recv.permute(1, 2, 0, 3, 4).reshape(B, Hl, P * Sl, D)


def heads_to_seq(x: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse of :func:`seq_to_heads`: ``[B, H/P, S, D]`` -> ``[B, H, S/P, D]``."""
    P = _world(group)
    if P == 1:
        if out is not None:
            out.copy_(x)
            return out
        return x
    B, Hl, S, D = x.shape
    if S % P:
        raise ValueError(f"sequence {S} does not divide over {P} ranks")
    Sl = S // P
    send = x.reshape(B, Hl, P, Sl, D).permute(2, 0, 1, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[r] holds rank r's heads for my sequence shard
    res = recv.permute(1, 0, 2, 3, 4).reshape(B, P * Hl, Sl, D)
    if out is not None:
        out.copy_(res)
        return out
    return res


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, kv_len=None, scale: Optional[float] = None,
                      group=None, out: Optional[torch.Tensor] = None, use_fixed_m: bool = False,
                      attend: Optional[Callable] = None) -> torch.Tensor:
    """Head-parallel attention on a sequence-sharded stream; ``kv_len`` holds global lengths."""
    attend = attend or ops.attention
    qh, kh, vh = seq_to_heads(q, group), seq_to_heads(k, group), seq_to_heads(v, group)
    oh = attend(qh, kh, vh, kv_len=kv_len, scale=scale, use_fixed_m=use_fixed_m)
    return heads_to_seq(oh, group, out=out)


def ring_schedule(rank: int, world: int) -> List[int]:
    """Origin rank of the K/V shard a rank holds at each ring step (step 0 is its own)."""
    return [(rank - t) % world for t in range(world)]


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, kv_len=None, scale: Optional[float] = None,
                   group=None, out: Optional[torch.Tensor] = None, use_fixed_m: bool = False,
                   mk: Optional[torch.Tensor] = None, zero_padded_rows: bool = True,
                   new_state: Optional[Callable] = None, fold: Optional[Callable] = None,
                   finalize: Optional[Callable] = None) -> torch.Tensor:
    """Ring-KV sequence-parallel attention: ``q, k, v`` are ``[B, H, S/P, D]`` shards in rank order.

    Step ``t`` folds the shard that originated on rank ``(rank - t) % P`` while the next shard is already
    in flight to this rank (double-buffered receive), so the transfer hides behind the kernel.
    """
    P, rank = _world(group), _rank(group)
    B, H, Sl, D = q.shape
    new_state = new_state or (lambda: ops.ResidualState(B, H, Sl, q.device))
    fold = fold or ops.residual_attention_
    finalize = finalize or ops.finalize_residual
    state = new_state()
    k_cur, v_cur = k.contiguous(), v.contiguous()
    bufs = [(torch.empty_like(k_cur), torch.empty_like(v_cur)) for _ in range(2)] if P > 1 else []
    ranks = dist.get_process_group_ranks(group) if (P > 1 and group is not None) else list(range(P))
    nxt, prv = ranks[(rank + 1) % P], ranks[(rank - 1) % P]
    for t, origin in enumerate(ring_schedule(rank, P)):
        reqs = []
        if t + 1 < P:
            k_nxt, v_nxt = bufs[t % 2]
            ops_list = [dist.P2POp(dist.isend, k_cur, nxt, group), dist.P2POp(dist.isend, v_cur, nxt, group),
                        dist.P2POp(dist.irecv, k_nxt, prv, group), dist.P2POp(dist.irecv, v_nxt, prv, group)]
            reqs = dist.batch_isend_irecv(ops_list)
        fold(state, q, k_cur, v_cur, scale=scale, kv_len=kv_len, kv_offset=origin * Sl, q_offset=rank * Sl,
             use_fixed_m=use_fixed_m, mk=mk)
        for r in reqs:
            r.wait()
        if t + 1 < P:
            k_cur, v_cur = k_nxt, v_nxt
    return finalize(state, kv_len=kv_len, q_offset=rank * Sl, zero_padded_rows=zero_padded_rows, out=out)


def make_sequence_shard(cfg, call_index: int, rank: int, world: int, device, base_seed: int = 0):
    """Rank ``rank``'s ``[B, H, S/P, D]`` shard of a seeded synthetic call, generated on ``device``.

    Each shard has its own Philox stream (seed ``1000*base + 8*call + rank``), so no rank ever
    materialises the whole tensor; the padding draw is shared by all ranks.
    """
    from .inputs import _qk_norm

    S = cfg.seq
    if S % world:
        raise ValueError(f"sequence {S} does not divide over {world} ranks")
    Sl = S // world
    g = torch.Generator(device=device).manual_seed(1000 * base_seed + 8 * call_index + rank)
    shape = (cfg.batch, cfg.heads, Sl, cfg.head_dim)
    q = _qk_norm(torch.randn(shape, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)
    k = _qk_norm(torch.randn(shape, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)
    v = torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    gp = torch.Generator(device="cpu").manual_seed(1_000_003 * (base_seed + call_index) + 17)
    pad = torch.randint(0, cfg.max_pad + 1, (cfg.batch,), generator=gp).clamp(max=cfg.text_tokens)
    kv_len = (S - pad).to(torch.int32).to(device)
    return q, k, v, kv_len
