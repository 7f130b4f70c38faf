"""dtb200 — B200-native joint (text + image/video token) attention forward for DiT blocks.

A drop-in for the device-local attention entry points of shungcp/diffusers-tpu
(``diffusers_tpu.kernels.splash.attention`` / ``residual_attention`` and the SDPA callable of
``diffusers_tpu.kernels.mesh_attention``), backed by hand-written sm_100a kernels behind a C ABI.
"""
from . import fixed_m  # noqa: F401
from .ops import (  # noqa: F401
    FIXED_M_RING_SAFE_BOUND,
    FIXED_M_SAFE_BOUND,
    ResidualState,
    attention,
    check_device_status,
    finalize_residual,
    fixed_m_operands,
    BlockTable,
    make_block_table,
    qk_prepass,
    describe_launch,
    out_proj,
    out_proj_reduce_,
    sum_partials,
    smooth_k,
    quantize_e4m3,
    sparse_attention,
    residual_attention,
    residual_attention_,
    sdpa,
)

__all__ = [
    "attention", "residual_attention", "residual_attention_", "finalize_residual", "fixed_m_operands",
    "sdpa", "describe_launch", "qk_prepass", "out_proj", "out_proj_reduce_", "sum_partials", "smooth_k", "quantize_e4m3", "sparse_attention", "make_block_table", "BlockTable", "ResidualState", "check_device_status", "FIXED_M_SAFE_BOUND", "FIXED_M_RING_SAFE_BOUND",
]
