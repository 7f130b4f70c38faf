"""CPU oracle for the joint (text + image/video token) attention forward.

TEST INFRASTRUCTURE, NOT PRODUCT CODE: only the tests, the smoke check and the CPU-baseline leg of
the bench may import this module.  The product path never routes through it.

PARITY UNPINNED: the reference project ships no golden vectors, known-answer tests or fixtures
for this kernel, and its own implementation (JAX + Pallas for TPU) cannot be imported or run
where this repository is developed.  The oracle is therefore pinned only by (i) agreement between
its two independent formulations below on seeded inputs and (ii) the invariants the reference
documents (padding invariance, k-smoothing invariance, fixed-m == online, tile-size independence).

Two formulations:

* ``attention_fp32``      the parity target: fp32 softmax over ``scale * q k^T`` with keys at or past
                          ``kv_len`` masked, as the reference's own CPU path computes it
                          (diffusers_tpu/models/moss_image/jax_dit.py:183-187,
                          diffusers_tpu/models/minimax_h3/jax_dit.py:393-399,
                          diffusers_tpu/kernels/mesh_attention.py:59-69).
* ``attention_restated``  the reference kernel's arithmetic restated step by step with its rounding
                          points and tile order (diffusers_tpu/kernels/splash.py:115-375, 566-650):
                          bf16 rounding of q*scale and of (q*scale)*log2e, f32 QK^T, exp2, f32 row
                          sums from unrounded probabilities, bf16 probabilities into the PV product,
                          online or fixed-m softmax per head, last KV block always online.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

LOG2_E = 1.44269504                      # diffusers_tpu/kernels/fixed_m_bound.py:33-35
FIXED_M_RECENTER = 88.0                  # fixed_m_bound.py:37-40
FIXED_M_SAFE_BOUND = 213.0               # fixed_m_bound.py:42-45
FIXED_M_RING_SAFE_BOUND = FIXED_M_SAFE_BOUND / 2.0   # fixed_m_bound.py:47-53
MASK_VALUE = -0.7 * float(np.finfo(np.float32).max)  # splash.py:45

KvLen = Union[None, int, Sequence[int], torch.Tensor]


def _kv_len_list(kv_len: KvLen, batch: int, skv: int) -> list:
    if kv_len is None:
        return [skv] * batch
    if isinstance(kv_len, torch.Tensor):
        vals = [int(x) for x in kv_len.reshape(-1).tolist()]
    elif isinstance(kv_len, (int, np.integer)):
        vals = [int(kv_len)]
    else:
        vals = [int(x) for x in kv_len]
    if len(vals) == 1:
        vals = vals * batch
    assert len(vals) == batch
    return [max(0, min(v, skv)) for v in vals]


def block_mask(kv_table, seq_q: int, seq_kv: int, block_q: int, block_kv: int) -> torch.Tensor:
    """Boolean ``[seq_q, seq_kv]`` mask of the (query, key) pairs a block table visits
    (diffusers_tpu/kernels/sparse_splash.py: per query block the sorted list of key blocks)."""
    m = torch.zeros(seq_q, seq_kv, dtype=torch.bool)
    for qb, blocks in enumerate(kv_table):
        for kb in blocks:
            m[qb * block_q:(qb + 1) * block_q, kb * block_kv:(kb + 1) * block_kv] = True
    return m


def attention_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
                   kv_len: KvLen = None, zero_padded_rows: bool = True, rows: Optional[torch.Tensor] = None,
                   out_dtype: torch.dtype = torch.float32, mask=None) -> torch.Tensor:
    """fp32-softmax attention on CPU, one (batch, head) at a time to bound memory.

    ``mask`` (bool ``[Sq, Skv]``, or one per head) restricts the keys each query sees (block-sparse calls); queries
    that see no key give zeros.  ``rows`` (1-D long tensor) restricts the computation to those query rows (sampled-row
    checks of long sequences); the result then has ``len(rows)`` rows.  Query rows at or past
    ``kv_len[b]`` are zero when ``zero_padded_rows`` (the callers of the reference zero padded
    queries: diffusers_tpu/models/minimax_h3/jax_dit.py:374-381).
    """
    q, k, v = q.detach().cpu(), k.detach().cpu(), v.detach().cpu()
    B, H, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    group = H // Hkv
    s = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    lens = _kv_len_list(kv_len, B, Skv)
    ridx = torch.arange(Sq) if rows is None else rows.cpu().long()
    out = torch.zeros(B, H, len(ridx), v.shape[-1], dtype=torch.float32)
    for b in range(B):
        n = lens[b]
        if n == 0:
            continue
        for h in range(H):
            qf = q[b, h].index_select(0, ridx).float()
            kf = k[b, h // group, :n].float()
            vf = v[b, h // group, :n].float()
            logits = (qf @ kf.T) * s
            if mask is not None:
                mh = mask[h] if isinstance(mask, (list, tuple)) else mask
                mh = mh.index_select(0, ridx)[:, :n]
                logits = logits.masked_fill(~mh, float("-inf"))
                dead = ~mh.any(dim=-1)
                logits[dead] = 0.0
            p = torch.softmax(logits, dim=-1)
            o = p @ vf
            if mask is not None:
                o[dead] = 0
            if zero_padded_rows and kv_len is not None:
                o[ridx >= n] = 0
            out[b, h] = o
    return out.to(out_dtype)


def max_row_norm_per_head(x: torch.Tensor) -> torch.Tensor:
    """Max L2 row norm per head over batch and sequence, f32 (fixed_m_bound.py:57-73)."""
    return x.float().pow(2).sum(-1).sqrt().amax(dim=(0, 2))


def fixed_m_operands(q_scaled: torch.Tensor, k: torch.Tensor, *, gate: float = FIXED_M_SAFE_BOUND) -> torch.Tensor:
    """``(2, heads)``: row 0 = ceil(bound), row 1 = bound <= gate (fixed_m_bound.py:98-118)."""
    qn = max_row_norm_per_head(q_scaled)
    kn = max_row_norm_per_head(k)
    if kn.numel() != qn.numel():
        kn = kn.repeat_interleave(qn.numel() // kn.numel())
    bound = qn * kn
    return torch.stack([torch.ceil(bound), (bound <= gate).float()])


def ring_fixed_m_operands(qn_max: torch.Tensor, kn_max: torch.Tensor) -> torch.Tensor:
    """Ring variant: m = floor(106.5) for every head, gate halved (fixed_m_bound.py:121-155)."""
    bound = qn_max * kn_max
    m = torch.full_like(bound, float(math.floor(FIXED_M_RING_SAFE_BOUND)))
    return torch.stack([m, (bound <= FIXED_M_RING_SAFE_BOUND).float()])


def scale_query(q: torch.Tensor, scale: Optional[float]) -> torch.Tensor:
    """``(q * scale) * log2e`` with a bf16 rounding after each multiply (splash.py:607-609, 633)."""
    s = (1.0 / math.sqrt(q.shape[-1])) if scale is None else float(scale)
    q1 = (q.float() * s).to(q.dtype)
    return (q1.float() * LOG2_E).to(q.dtype).to(torch.bfloat16)


def smooth_keys(k: torch.Tensor, kv_len: KvLen = None) -> torch.Tensor:
    """Caller-side k-smoothing: ``k - mean_seq(k)`` over valid rows, padded rows zeroed.

    Unpadded form diffusers_tpu/kernels/mesh_attention.py:234-237; padded form with an f32 mean
    diffusers_tpu/models/minimax_h3/jax_server.py:276-281.
    """
    B, H, S, D = k.shape
    if kv_len is None:
        return k - k.mean(dim=2, keepdim=True)
    lens = _kv_len_list(kv_len, B, S)
    out = torch.zeros_like(k)
    for b in range(B):
        n = lens[b]
        if n == 0:
            continue
        mean = k[b, :, :n].float().sum(dim=1, keepdim=True) / n
        out[b, :, :n] = k[b, :, :n] - mean.to(k.dtype)
    return out


def _restated_one(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, m_fixed: Optional[float], kv_len: Optional[int],
                  bq: int, bkv: int, bkv_c: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One (batch, head): returns unnormalised o f32 [Sq, Dv], m [Sq], l [Sq] (splash.py:115-375)."""
    Sq, Skv = q.shape[0], k.shape[0]
    bq, bkv = min(bq, Sq), min(bkv, Skv)
    bkv_c = min(bkv_c, Skv)
    if bkv % bkv_c:
        bkv_c = bkv                                   # splash.py:555-558
    n_kv_blocks = (Skv + bkv - 1) // bkv
    qf, kf = q.float(), k.float()
    vb = v.to(torch.bfloat16).float()
    o = torch.zeros(Sq, v.shape[-1], dtype=torch.float32)
    m = torch.full((Sq,), MASK_VALUE if m_fixed is None else m_fixed - FIXED_M_RECENTER, dtype=torch.float32)
    l = torch.zeros(Sq, dtype=torch.float32)
    for i0 in range(0, Sq, bq):
        rows = slice(i0, min(i0 + bq, Sq))
        for j in range(n_kv_blocks):
            last = j == n_kv_blocks - 1
            blk_lo, blk_hi = j * bkv, min((j + 1) * bkv, Skv)
            has_pad = kv_len is not None and blk_hi > kv_len
            use_fixed = (m_fixed is not None) and not last and not has_pad       # splash.py:334-357
            for c0 in range(blk_lo, blk_hi, bkv_c):
                c1 = min(c0 + bkv_c, blk_hi)
                qk = qf[rows] @ kf[c0:c1].T                                      # f32 accumulate
                if kv_len is not None and (last or has_pad):
                    pos = torch.arange(c0, c1)
                    qk = torch.where(pos[None, :] < kv_len, qk, torch.tensor(MASK_VALUE))
                if use_fixed:
                    s = torch.exp2(qk - m[rows, None])
                    l[rows] = l[rows] + s.sum(-1)
                    o[rows] = o[rows] + s.to(torch.bfloat16).float() @ vb[c0:c1]
                else:
                    m_prev = m[rows]
                    m_next = torch.maximum(m_prev, qk.max(-1).values)
                    s = torch.exp2(qk - m_next[:, None])
                    alpha = torch.exp2(m_prev - m_next)
                    l[rows] = alpha * l[rows] + s.sum(-1)
                    o[rows] = alpha[:, None] * o[rows] + s.to(torch.bfloat16).float() @ vb[c0:c1]
                    m[rows] = m_next
    return o, m, l


def attention_restated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
                       kv_len: Optional[int] = None, block_q: int = 1024, block_kv: int = 2048,
                       block_kv_compute: int = 1024, use_fixed_m: bool = False, emit_residuals: bool = False,
                       mk: Optional[torch.Tensor] = None):
    """The reference kernel's arithmetic on CPU (one scalar ``kv_len`` per call, as there).

    Returns the normalised output in ``q``'s dtype, or ``(o_unnorm f32, m, l)`` with ``m``/``l`` of
    shape ``[B,H,Sq,1]`` when ``emit_residuals`` (splash.py:665-742).
    """
    q, k, v = q.detach().cpu(), k.detach().cpu(), v.detach().cpu()
    B, H, Sq, D = q.shape
    group = H // k.shape[1]
    qs = scale_query(q, scale)
    if use_fixed_m and mk is None:
        mk = fixed_m_operands(qs, k)
    out = torch.zeros(B, H, Sq, v.shape[-1], dtype=torch.float32)
    ms = torch.zeros(B, H, Sq, dtype=torch.float32)
    ls = torch.zeros(B, H, Sq, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            m_fixed = None
            if use_fixed_m and float(mk[1, h]) > 0.5:
                m_fixed = float(mk[0, h])
            o, m, l = _restated_one(qs[b, h], k[b, h // group], v[b, h // group], m_fixed, kv_len, block_q, block_kv,
                                    block_kv_compute)
            out[b, h], ms[b, h], ls[b, h] = o, m, l
    if emit_residuals:
        return out, ms.unsqueeze(-1), ls.unsqueeze(-1)
    return (out * (1.0 / ls).unsqueeze(-1)).to(q.dtype)


def merge_residuals(parts: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]) -> torch.Tensor:
    """LSE-space merge of ring partials: ``sum_i o_i 2^(m_i-M) / sum_i l_i 2^(m_i-M)`` (splash.py:657-662)."""
    ms = torch.stack([p[1].reshape(p[0].shape[:-1]) for p in parts])
    ls = torch.stack([p[2].reshape(p[0].shape[:-1]) for p in parts])
    os_ = torch.stack([p[0] for p in parts])
    live = ls > 0
    M = torch.where(live, ms, torch.tensor(-float("inf"))).amax(dim=0)
    w = torch.where(live, torch.exp2(ms - M), torch.zeros(()))
    L = (w * ls).sum(0)
    O = (w.unsqueeze(-1) * os_).sum(0)
    return torch.where(L.unsqueeze(-1) > 0, O / L.unsqueeze(-1), torch.zeros(()))


def qk_prepass(q: torch.Tensor, k: torch.Tensor, v: Optional[torch.Tensor] = None, *, q_weight=None, k_weight=None,
               eps: float = 1e-5, rope=None, kv_len: KvLen = None):
    """The block-level steps in front of the kernel, on CPU: RMSNorm per head, rotary embedding, pad zeroing and
    the ``(B, S, H, D) -> (B, H, S, D)`` swap (diffusers_tpu/models/minimax_h3/jax_dit.py:191-195, 251-262, 362-388).

    The norm is computed in f32 and cast to the input dtype; the rotation is applied to those bf16 values with the
    tables cast to bf16, in f32 with one final rounding (the reference rounds after each bf16 operation on some
    backends, which moves results by at most one bf16 ulp).
    """
    def norm(x, w):
        x32 = x.float()
        y = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
        if w is not None:
            y = y * w.float()
        return y.to(x.dtype)

    def turn(x, cos, sin):
        rotary = cos.shape[-1]
        rotated, passed = x[..., :rotary].float(), x[..., rotary:]
        c = cos.to(x.dtype).float()[None, :, None, :]
        s = sin.to(x.dtype).float()[None, :, None, :]
        x1, x2 = rotated.chunk(2, dim=-1)
        turned = torch.cat([-x2, x1], dim=-1)
        return torch.cat([(rotated * c + turned * s).to(x.dtype), passed], dim=-1)

    qn, kn = norm(q, q_weight), norm(k, k_weight)
    if rope is not None:
        qn, kn = turn(qn, *rope), turn(kn, *rope)
    outs = [qn, kn] + ([v] if v is not None else [])
    if kv_len is not None:
        lens = _kv_len_list(kv_len, q.shape[0], q.shape[1])
        keep = (torch.arange(q.shape[1])[None, :] < torch.tensor(lens)[:, None])[:, :, None, None]
        outs = [torch.where(keep, t, torch.zeros((), dtype=t.dtype)) for t in outs]
    outs = [t.transpose(1, 2).contiguous() for t in outs]
    return (outs[0], outs[1], outs[2] if v is not None else None)


def out_proj(o: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``to_out`` behind head-major attention output: f32 ``[B, S, N]`` from ``o`` ``[B, H, S, D]`` and the ``[H*D, N]``
    rows of the weight for those heads; a partial sum when the heads are a shard
    (diffusers_tpu/models/minimax_h3/jax_image_pipeline.py:574-593)."""
    B, H, S, D = o.shape
    x = o.detach().cpu().float().permute(0, 2, 1, 3).reshape(B, S, H * D)
    return x @ w.detach().cpu().float()
