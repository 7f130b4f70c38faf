"""Seeded synthetic stand-ins for DiT attention activations.

The reference measures on real prompts and latents, which are not available offline; these
generators reproduce the shapes and value distribution the benchmark configurations name:
q, k, v ~ N(0,1), per-head RMSNorm with unit weight on q and k (the qk-norm of
``diffusers_tpu/models/moss_image/jax_dit.py:126-129``, eps 1e-6), cast to bf16, sequence laid out
``[image/video tokens | text tokens]`` with padding as trailing text tokens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class AttnConfig:
    name: str
    batch: int
    heads: int
    media_tokens: int
    text_tokens: int
    head_dim: int = 128
    max_pad: int = 300          # padding per batch element is drawn from [0, max_pad]
    fixed_pad: Optional[int] = None

    @property
    def seq(self) -> int:
        return self.media_tokens + self.text_tokens

    def flops(self) -> float:
        """4 * B * H * Sq * Sk * D, padded keys included (the metric's definition)."""
        return 4.0 * self.batch * self.heads * self.seq * self.seq * self.head_dim


CONFIGS = {
    "c1_image512_cpu": AttnConfig("c1_image512_cpu", 1, 24, 1024, 256, fixed_pad=37),
    "c2_image1024": AttnConfig("c2_image1024", 2, 24, 4096, 512),
    "c3_image2048": AttnConfig("c3_image2048", 2, 24, 16384, 512),
    "c4_video480p": AttnConfig("c4_video480p", 2, 40, 48360, 512),
    "c5_video768p": AttnConfig("c5_video768p", 1, 40, 350784, 512),
}


def _qk_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def make_inputs(cfg: AttnConfig, call_index: int = 0, base_seed: int = 0, device: str = "cpu",
                heads: Optional[int] = None, seq: Optional[int] = None
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns bf16 ``q, k, v`` of shape ``[B, H, S, D]`` and int32 ``kv_len`` of shape ``[B]``.

    The generator is seeded with ``base_seed + call_index`` on ``device`` (CPU streams are shared
    bit-for-bit with the CPU oracle; CUDA streams are used for the shapes too large to ship).
    ``heads`` / ``seq`` override the configured sizes for shards and reduced test cases.
    """
    H = cfg.heads if heads is None else heads
    S = cfg.seq if seq is None else seq
    g = torch.Generator(device=device).manual_seed(base_seed + call_index)
    shape = (cfg.batch, H, S, cfg.head_dim)
    q = _qk_norm(torch.randn(shape, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)
    k = _qk_norm(torch.randn(shape, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)
    v = torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    if cfg.fixed_pad is not None:
        pad = torch.full((cfg.batch,), cfg.fixed_pad, dtype=torch.int64)
    else:
        gp = torch.Generator(device="cpu").manual_seed(1_000_003 * (base_seed + call_index) + 17)
        pad = torch.randint(0, cfg.max_pad + 1, (cfg.batch,), generator=gp)
    pad = pad.clamp(max=max(min(cfg.text_tokens, S - 1), 0))
    kv_len = (S - pad).to(torch.int32).to(device)
    return q, k, v, kv_len
