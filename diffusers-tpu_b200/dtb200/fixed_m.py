"""Host-side derivation of the bounded-logit ("fixed-m") softmax operand.

Mirrors ``diffusers_tpu/kernels/fixed_m_bound.py``: the safety constants, the per-head Cauchy-Schwarz bound from row
norms, its ring variant, the sampled measurement of the true max logit used for offline calibration, and the builder
that turns calibrated norms into the ``(2, heads)`` operand the kernel consumes (row 0 = integral ``m``, row 1 =
eligibility).  Everything here is ordinary PyTorch/NumPy that runs off the hot path, on CPU or GPU tensors; the
per-call bound of the hot path is computed by the CUDA kernels behind ``dtb200.fixed_m_operands`` /
``dtb200.qk_prepass``.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

# The kernels exponentiate with exp2, so logits are measured in log2 units (fixed_m_bound.py:33-35).
LOG2_E = 1.44269504
# s = exp2(qk - m + 88): the recentring that maximises the no-flush window (fixed_m_bound.py:37-40).
FIXED_M_RECENTER = 88.0
# A head may use the constant offset only if its bound is <= 213: the flush gap then stays below 88 + 126
# (fixed_m_bound.py:42-45).
FIXED_M_SAFE_BOUND = 213.0
# Ring shards see un-smoothed keys, so only |qk| <= bound holds and the gate halves (fixed_m_bound.py:47-53).
FIXED_M_RING_SAFE_BOUND = FIXED_M_SAFE_BOUND / 2.0
# Query rows visited when measuring the true max logit (fixed_m_bound.py:156-165).
MAX_LOGIT_SAMPLE_ROWS = 1024
# E4M3 rounding can raise a magnitude by up to 2^-4, on q and on k (fixed_m_bound.py:293-297).
_QK_FP8_BOUND_INFLATION = (1.0 + 2.0 ** -4) ** 2
_E4M3_MAX = 448.0


def _seq_dims(seq_axis: int):
    if seq_axis not in (1, 2):
        raise ValueError(f"seq_axis must be 1 or 2, got {seq_axis}")
    return (0, seq_axis)


def max_row_norm_per_head(x: torch.Tensor, *, seq_axis: int = 2) -> torch.Tensor:
    """``(heads,)`` f32: the largest L2 row norm of each head over batch and sequence (fixed_m_bound.py:57-73)."""
    return x.float().pow(2).sum(-1).sqrt().amax(dim=_seq_dims(seq_axis))


def fixed_m_query_norms(query: torch.Tensor, scale: Optional[float] = None, *, seq_axis: int = 2) -> torch.Tensor:
    """Largest row norm of ``query * scale * log2(e)`` per head, the scale folded in as a scalar
    (fixed_m_bound.py:76-95)."""
    s = 1.0 / math.sqrt(query.shape[-1]) if scale is None else scale
    return max_row_norm_per_head(query, seq_axis=seq_axis) * (s * LOG2_E)


def fixed_m_operands(query_scaled: torch.Tensor, key: torch.Tensor, *, gate: float, seq_axis: int = 2) -> torch.Tensor:
    """``(2, heads)``: row 0 = ceil(Cauchy-Schwarz bound), row 1 = bound <= gate (fixed_m_bound.py:98-118)."""
    qn = max_row_norm_per_head(query_scaled, seq_axis=seq_axis)
    kn = max_row_norm_per_head(key, seq_axis=seq_axis)
    if kn.numel() != qn.numel():
        kn = kn.repeat_interleave(qn.numel() // kn.numel())
    bound = qn * kn
    return torch.stack([torch.ceil(bound), (bound <= gate).float()])


def ring_fixed_m_operands(qn_max: torch.Tensor, mk_h: torch.Tensor) -> torch.Tensor:
    """The ring's runtime operand from norms it already carries: the same ``m = floor(106.5)`` for every head and
    the halved gate on ``qn_max * mk_h`` (fixed_m_bound.py:121-155).  ``m`` cancels in ``o / l`` and an eligible head
    has a flush gap of at most 212.5 < 214, so one constant row is both safe and off the critical path."""
    bound = qn_max.float() * mk_h.float()
    m = torch.full_like(bound, float(math.floor(FIXED_M_RING_SAFE_BOUND)))
    return torch.stack([m, (bound <= FIXED_M_RING_SAFE_BOUND).float()])


def quantize_saturating(x: torch.Tensor) -> torch.Tensor:
    """Saturating cast to E4M3 (``diffusers_tpu/kernels/fp8_cast.py:28-39``): clamp to +-448, then round."""
    return x.float().clamp(-_E4M3_MAX, _E4M3_MAX).to(torch.float8_e4m3fn)


def sampled_max_abs_logit(query: torch.Tensor, key: torch.Tensor, scale: Optional[float] = None, *, seq_axis: int = 2,
                          num_samples: int = MAX_LOGIT_SAMPLE_ROWS, qk_fp8: bool = False, rows_per_chunk: int = 64,
                          group=None) -> torch.Tensor:
    """``(heads,)`` f32 max ``|q . k| * scale * log2(e)`` over a strided sample of query rows and ALL key rows.

    Follows fixed_m_bound.py:169-290: the stride is ``ceil(seq / num_samples)`` so the tail of the sequence is always
    visited; the sampled rows are scaled and rounded to bf16 (and both operands through E4M3 when ``qk_fp8``) so the
    measured logits are the ones the kernel forms; scores are taken ``rows_per_chunk`` query rows at a time.
    ``num_samples <= 0`` or ``>= seq`` visits every row (exact).  With ``group`` (sequence-sharded ranks), the
    sampled rows of all ranks are gathered so every rank scores them against its own key shard, and the per-head
    maxima are reduced with MAX over the group — the all-gather / pmax pair of the reference.
    """
    if seq_axis == 2:
        query, key = query.transpose(1, 2), key.transpose(1, 2)
    elif seq_axis != 1:
        raise ValueError(f"seq_axis must be 1 or 2, got {seq_axis}")
    seq, heads, dim = query.shape[1], query.shape[2], query.shape[3]
    s = 1.0 / math.sqrt(dim) if scale is None else scale
    wanted = seq if num_samples <= 0 or num_samples >= seq else num_samples
    stride = -(-seq // wanted)
    sample = query[:, ::stride].contiguous()
    if group is not None and dist.get_world_size(group) > 1:
        parts = [torch.empty_like(sample) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, sample, group=group)
        sample = torch.cat(parts, dim=1)
    sample = (sample.float() * (s * LOG2_E)).to(torch.bfloat16)
    keys = key.to(torch.bfloat16)
    if qk_fp8:
        sample = quantize_saturating(sample).to(torch.bfloat16)
        keys = quantize_saturating(keys).to(torch.bfloat16)
    kh = keys.float().permute(0, 2, 3, 1)                    # (B, H, D, seq)
    best = torch.zeros(heads, dtype=torch.float32, device=query.device)
    for r0 in range(0, sample.shape[1], max(1, rows_per_chunk)):
        block = sample[:, r0:r0 + rows_per_chunk].float().permute(0, 2, 1, 3)   # (B, H, rows, D)
        scores = torch.matmul(block, kh)                     # (B, H, rows, seq), f32 accumulate
        best = torch.maximum(best, scores.abs().amax(dim=(0, 2, 3)))
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(best, op=dist.ReduceOp.MAX, group=group)
    return best


def static_fixed_m_operands(qn_max, mk_h, *, margin_log2: float, qk_fp8: bool = False,
                            gate: float = FIXED_M_RING_SAFE_BOUND, max_logit=None) -> np.ndarray:
    """``(2, heads)`` f32 operand from CALIBRATED norms (fixed_m_bound.py:300-408).

    Row 0 is ``floor(gate)`` for every head — the largest ``m`` the gate permits, so that a head whose true bound
    drifts fails gracefully (a ring step underflows to zero weight at ``214 - floor(gate)``) before it can overflow
    (at ``floor(gate) + 16``).  Row 1 is ``ceil(bound) + margin_log2 <= gate`` where ``bound`` is the Cauchy-Schwarz
    product (inflated by ``(1 + 2^-4)^2`` under ``qk_fp8``) intersected with the measured ``max_logit`` when given.
    Raises ``ValueError`` for mismatched or non-1-D norms, a negative margin, or a ``max_logit`` that is not a finite
    non-negative ``(heads,)`` array.
    """
    qn = np.asarray(qn_max, dtype=np.float64)
    kn = np.asarray(mk_h, dtype=np.float64)
    if qn.ndim != 1 or qn.shape != kn.shape:
        raise ValueError(f"expected matching 1-D (heads,) norms, got {qn.shape} and {kn.shape}")
    if margin_log2 < 0.0:
        raise ValueError(f"margin_log2 must be >= 0, got {margin_log2}")
    bound = qn * kn
    if qk_fp8:
        bound = bound * _QK_FP8_BOUND_INFLATION
    if max_logit is not None:
        measured = np.asarray(max_logit, dtype=np.float64)
        if measured.shape != bound.shape:
            raise ValueError(f"max_logit must be {bound.shape}, got {measured.shape}")
        if not np.all(np.isfinite(measured)) or np.any(measured < 0.0):
            raise ValueError("max_logit must be finite and non-negative")
        bound = np.minimum(bound, measured)
    flag = (np.ceil(bound) + margin_log2 <= gate).astype(np.float64)
    m = np.full_like(bound, np.floor(gate))
    return np.stack([m, flag]).astype(np.float32)
