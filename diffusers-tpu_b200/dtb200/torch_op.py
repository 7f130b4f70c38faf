"""The attention registered as a torch custom op, and the diffusers dispatch hook.

Mirrors ``diffusers_tpu/backends/ours_splash_tt.py``: ``_op_for`` registers
``fn(query, key, value) -> out`` with a fake kernel returning ``empty_like(query)`` (``:45-77``) so the op
traces under ``torch.compile`` without running; ``install`` patches
``diffusers.models.attention_dispatch.dispatch_attention_fn`` and falls back to the original function for
masks, dropout, causal calls and short sequences (``:95-152``).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import ops

MIN_SEQ = int(os.environ.get("DTB_MIN_SEQ", "1024"))   # shorter sequences keep the stock path (ours_splash_tt.py:31-39)


@torch.library.custom_op("dtb200::joint_attention", mutates_args=(), device_types="cuda")
def joint_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    kv_len: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """``[B, H, S, D]`` bf16 in, same shape and dtype out; ``kv_len`` int32 ``[B]`` or ``[1]``."""
    return ops.attention(query, key, value, kv_len=kv_len, scale=scale)


@joint_attention.register_fake
def _(query, key, value, kv_len=None, scale=None):
    return torch.empty_like(query, memory_format=torch.contiguous_format)


@torch.library.custom_op("dtb200::joint_attention_fixed_m", mutates_args=(), device_types="cuda")
def joint_attention_fixed_m(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                            kv_len: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """The bounded-logit variant together with the k-smoothing it presumes (``ours_splash_tt.py:126-137``)."""
    return ops.sdpa(query, key, value, scale=scale, kv_len=kv_len, use_fixed_m=True)


@joint_attention_fixed_m.register_fake
def _(query, key, value, kv_len=None, scale=None):
    return torch.empty_like(query, memory_format=torch.contiguous_format)


FIXED_M = os.environ.get("DTB_FIXED_M", "0") == "1"   # the reference's torch backend runs use_fixed_m=True with smoothed keys


_original_dispatch = None


def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, _already_bhsd=False,
             **kwargs):
    """Replacement for diffusers' ``dispatch_attention_fn``: ``(B, seq, heads, dim)`` in and out."""
    seq = query.shape[2] if _already_bhsd else query.shape[1]
    unsupported = (attn_mask is not None or dropout_p != 0.0 or is_causal or seq < MIN_SEQ
                   or query.dtype != torch.bfloat16 or query.shape[-1] != 128 or not query.is_cuda)
    if unsupported:
        if _original_dispatch is None:
            raise NotImplementedError("this call needs the stock attention path, which is not installed")
        return _original_dispatch(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                  scale=scale, **kwargs)
    if not _already_bhsd:
        query, key, value = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    op = torch.ops.dtb200.joint_attention_fixed_m if FIXED_M else torch.ops.dtb200.joint_attention
    out = op(query, key, value, None, scale)
    return out if _already_bhsd else out.transpose(1, 2)


def install() -> bool:
    """Patches diffusers' attention dispatch; returns False when diffusers is not importable (``:85-90``)."""
    global _original_dispatch
    try:
        from diffusers.models import attention_dispatch
    except Exception:
        return False
    if _original_dispatch is None:
        _original_dispatch = attention_dispatch.dispatch_attention_fn
    attention_dispatch.dispatch_attention_fn = dispatch
    return True
