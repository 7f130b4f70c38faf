"""Device-local joint attention: the host-side mirror of the reference's kernel entry points.

``attention`` and ``residual_attention`` keep the keyword surface of
``diffusers_tpu/kernels/splash.py:566-650`` and ``:665-742`` (``query, key, value`` laid out
``[B, heads, seq, dim]``, ``scale=None`` meaning ``1/sqrt(dim)``, output in ``query``'s dtype);
``sdpa`` keeps the SDPA signature of ``diffusers_tpu/kernels/mesh_attention.py:218-228``
(the mask / dropout / causal / gqa arguments are accepted and ignored, as there).
Tile-size keywords of the reference are accepted and ignored: tiling is fixed by the kernel.

All compute goes through the C ABI in ``libdtb200_attn.so``; nothing here falls back to PyTorch.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence, Tuple, Union

import torch

from . import _lib

LOG2_E = 1.44269504
FIXED_M_SAFE_BOUND = 213.0        # diffusers_tpu/kernels/fixed_m_bound.py:44-47
FIXED_M_RING_SAFE_BOUND = 106.5   # diffusers_tpu/kernels/fixed_m_bound.py:49-54

KvLen = Union[None, int, Sequence[int], torch.Tensor]

_status_bufs: dict = {}
_workspaces: dict = {}


def _status_buffer(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    buf = _status_bufs.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=device)
        _status_bufs[key] = buf
    return buf


def _workspace(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Split-KV scratch, one buffer per (device, stream): calls on different streams may overlap on the GPU."""
    if nbytes == 0:
        return None
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def check_device_status(device: Union[torch.device, str, None] = None) -> None:
    """Synchronises ``device`` and raises if a kernel reported a bounded wait that ran out."""
    device = torch.device(device if device is not None else "cuda")
    torch.cuda.synchronize(device)
    buf = _status_buffer(device)
    st = buf.tolist()
    if st[0] != 0:
        buf.zero_()
        raise RuntimeError(
            f"dtb200 kernel error {st[0]} (1 = wait timeout) at site {st[1]}, CTA {st[2]}, detail {st[3]}"
        )


def _check_inputs(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> None:
    for name, t in (("query", query), ("key", key), ("value", value)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: dtb200 has no CPU path")
        if t.dtype != torch.bfloat16:
            raise NotImplementedError(f"{name} must be bfloat16, got {t.dtype}")
        if t.dim() != 4:
            raise ValueError(f"{name} must be [B, heads, seq, dim], got shape {tuple(t.shape)}")
    if query.shape[-1] != 128 or key.shape[-1] != 128 or value.shape[-1] != 128:
        raise NotImplementedError("head_dim must be 128")
    if key.shape != value.shape:
        raise ValueError("key and value must have the same shape")
    if query.shape[0] != key.shape[0]:
        raise ValueError("batch sizes differ")
    if query.shape[1] % key.shape[1] != 0:
        raise ValueError("query heads must be a multiple of key/value heads")


def _dense_last(t: torch.Tensor) -> torch.Tensor:
    """Returns ``t`` if the kernel can address it in place (contiguous head_dim, 16-byte strides)."""
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(
        n == 1 or (s > 0 and (s * 2) % 16 == 0) for n, s in zip(t.shape[:-1], t.stride()[:-1]))
    return t if ok else t.contiguous()   # broadcast (stride 0) and odd-stride views are materialised


def _kv_len_tensor(kv_len: KvLen, batch: int, device: torch.device) -> Optional[torch.Tensor]:
    if kv_len is None:
        return None
    if isinstance(kv_len, torch.Tensor):
        t = kv_len.to(device=device, dtype=torch.int32).reshape(-1)
        if t.numel() == 1 and batch > 1:
            t = t.expand(batch)
        if t.numel() != batch:
            raise ValueError(f"kv_len must have 1 or {batch} entries, got {t.numel()}")
        return t.contiguous()
    if isinstance(kv_len, (list, tuple)):
        return _kv_len_tensor(torch.tensor(list(kv_len), dtype=torch.int32), batch, device)
    return torch.full((batch,), int(kv_len), dtype=torch.int32, device=device)


def _fill_params(query, key, value, out, kv_len_t, mk, scale, flags, num_splits, status) -> _lib.AttnParams:
    p = _lib.AttnParams()
    p.q, p.k, p.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    p.o = out.data_ptr() if out is not None else None
    p.B, p.Hq, p.Sq, p.D = query.shape[0], query.shape[1], query.shape[2], query.shape[3]
    p.Hkv, p.Skv = key.shape[1], key.shape[2]
    p.q_stride_b, p.q_stride_h, p.q_stride_s = query.stride()[:3]
    p.k_stride_b, p.k_stride_h, p.k_stride_s = key.stride()[:3]
    p.v_stride_b, p.v_stride_h, p.v_stride_s = value.stride()[:3]
    if out is not None:
        p.o_stride_b, p.o_stride_h, p.o_stride_s = out.stride()[:3]
    p.kv_len = kv_len_t.data_ptr() if kv_len_t is not None else None
    p.mk = mk.data_ptr() if mk is not None else None
    p.scale = float(scale) if scale is not None else 0.0
    p.flags = flags
    p.num_splits = int(num_splits)
    p.status = status.data_ptr() if status is not None else None
    return p


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def fixed_m_operands(query: torch.Tensor, key: torch.Tensor, *, scale: Optional[float] = None,
                     gate: float = FIXED_M_SAFE_BOUND) -> torch.Tensor:
    """``(2, heads)`` f32 bounded-logit operand: row 0 = ceil(Cauchy-Schwarz bound), row 1 = eligibility.

    Mirrors ``fixed_m_bound.fixed_m_operands`` over ``fixed_m_query_norms``
    (``diffusers_tpu/kernels/fixed_m_bound.py:76-118``): the bound is the product of the largest
    scaled query row norm and the largest key row norm of each head, over batch and sequence.
    """
    _check_inputs(query, key, key)
    query, key = _dense_last(query), _dense_last(key)
    dev = query.device
    norms = torch.empty(query.shape[1] + key.shape[1], dtype=torch.float32, device=dev)
    mk = torch.empty(2, query.shape[1], dtype=torch.float32, device=dev)
    p = _fill_params(query, key, key, None, None, None, scale, 0, 1, None)
    with torch.cuda.device(dev):
        st = _lib.load().dtb_fixed_m_operands(ctypes.byref(p), float(gate), norms.data_ptr(), mk.data_ptr(),
                                              _stream_ptr(dev))
    _lib.check(st, "dtb_fixed_m_operands")
    return mk


def row_norm_maxima(query: torch.Tensor, key: torch.Tensor, *, scale: Optional[float] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(heads_q,)`` largest row norm of ``query * scale * log2(e)`` and ``(heads_kv,)`` largest key row norm, f32,
    over batch and sequence (``fixed_m_query_norms`` / ``max_row_norm_per_head``,
    ``diffusers_tpu/kernels/fixed_m_bound.py:57-95``): the two factors a sequence-parallel caller reduces with
    MAX over its ranks before it forms the ring operand."""
    _check_inputs(query, key, key)
    query, key = _dense_last(query), _dense_last(key)
    dev = query.device
    norms = torch.empty(query.shape[1] + key.shape[1], dtype=torch.float32, device=dev)
    mk = torch.empty(2, query.shape[1], dtype=torch.float32, device=dev)
    p = _fill_params(query, key, key, None, None, None, scale, 0, 1, None)
    with torch.cuda.device(dev):
        st = _lib.load().dtb_fixed_m_operands(ctypes.byref(p), float(FIXED_M_SAFE_BOUND), norms.data_ptr(),
                                              mk.data_ptr(), _stream_ptr(dev))
    _lib.check(st, "dtb_fixed_m_operands")
    return norms[:query.shape[1]], norms[query.shape[1]:]


def quantize_e4m3(x: torch.Tensor, *, mult: float = 1.0) -> torch.Tensor:
    """Saturating E4M3 cast of a bf16 ``[B, H, S, 128]`` tensor: ``x * mult`` clamped to +-448, as
    ``diffusers_tpu/kernels/fp8_cast.py:28-39``.  Returns contiguous ``torch.float8_e4m3fn``."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 4 or x.shape[-1] != 128:
        raise NotImplementedError("quantize_e4m3 takes CUDA bf16 [B, H, S, 128] tensors")
    x = _dense_last(x)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().dtb_quantize_e4m3(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), x.shape[0], x.shape[1],
                                           x.shape[2], x.shape[3], float(mult), out.data_ptr(), _stream_ptr(x.device))
    _lib.check(st, "dtb_quantize_e4m3")
    return out.view(torch.float8_e4m3fn)


def _smooth_k(key: torch.Tensor, *, kv_len: KvLen = None, out: Optional[torch.Tensor] = None,
              want_norms: bool = False):
    """k-smoothing: ``key - mean_seq(key)`` over the valid rows of each (batch, head), padded rows zeroed.

    The caller-side preconditioning of ``diffusers_tpu/kernels/mesh_attention.py:234-237`` (unpadded) and
    ``diffusers_tpu/models/minimax_h3/jax_server.py:276-281`` (padded: f32 sum over the kept rows divided by
    ``kv_len``, mean rounded to the key dtype, pads written as zeros).  Softmax is invariant to it; it makes
    every query row's largest logit non-negative, which the bounded-logit softmax's wide gate presumes.
    ``out`` may be ``key`` (in place).  With ``want_norms`` also returns the ``[H]`` f32 largest output row
    norm per head.
    """
    if not key.is_cuda:
        raise RuntimeError("key must be a CUDA tensor: dtb200 has no CPU path")
    if key.dtype != torch.bfloat16 or key.dim() != 4 or key.shape[-1] != 128:
        raise NotImplementedError(f"smooth_k takes bf16 [B, H, S, 128] tensors, got {key.dtype} {tuple(key.shape)}")
    if key.stride(-1) != 1 or key.data_ptr() % 16 or any(st % 8 for st in key.stride()[:3]):
        key = key.contiguous()
    B, H, S, _ = key.shape
    dev = key.device
    if out is None:
        out = torch.empty((B, H, S, 128), dtype=torch.bfloat16, device=dev)
    lib = _lib.load()
    scratch = torch.empty(lib.dtb_smooth_k_scratch_bytes(B, H), dtype=torch.uint8, device=dev)
    norms = torch.empty(H, dtype=torch.float32, device=dev) if want_norms else None
    kv_len_t = _kv_len_tensor(kv_len, B, dev)
    sp = _lib.SmoothKParams()
    sp.k = key.data_ptr()
    sp.k_stride_b, sp.k_stride_h, sp.k_stride_s = key.stride()[:3]
    sp.out = out.data_ptr()
    sp.out_stride_b, sp.out_stride_h, sp.out_stride_s = out.stride()[:3]
    sp.kv_len = kv_len_t.data_ptr() if kv_len_t is not None else None
    sp.scratch, sp.scratch_bytes = scratch.data_ptr(), scratch.numel()
    sp.k_norm_max = norms.data_ptr() if norms is not None else None
    sp.B, sp.H, sp.S, sp.D = B, H, S, 128
    with torch.cuda.device(dev):
        st = lib.dtb_smooth_k(ctypes.byref(sp), _stream_ptr(dev))
    _lib.check(st, "dtb_smooth_k")
    return (out, norms) if want_norms else out


smooth_k = _smooth_k   # public name; functions with a ``smooth_k`` flag call the underscored one


def attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    scale: Optional[float] = None,
    block_q: Optional[int] = None,
    block_kv: Optional[int] = None,
    block_kv_compute: Optional[int] = None,
    use_fixed_m: bool = False,
    qk_fp8: bool = False,
    kv_len: KvLen = None,
    kv_mask_all: bool = False,
    unroll: Optional[bool] = None,
    mk: Optional[torch.Tensor] = None,
    zero_padded_rows: bool = True,
    num_splits: int = 0,
    out: Optional[torch.Tensor] = None,
    k_smoothed: bool = False,
) -> torch.Tensor:
    """Normalised joint attention, ``(B, heads, seq_q, dim)`` in ``query``'s dtype.

    Same contract as ``diffusers_tpu/kernels/splash.py:566-650``.  ``kv_len`` may be an int, a
    0-d tensor (the reference's traced scalar) or a ``[B]`` tensor, which replaces the
    reference's per-sample Python loop (``diffusers_tpu/models/moss_image/jax_dit.py:199-203``).
    Keys at or past ``kv_len`` are masked; with ``zero_padded_rows`` query rows at or past it
    come back as exact zeros, so padding content cannot reach real rows or leak downstream.
    ``use_fixed_m`` selects the per-head constant-offset softmax for heads whose bound passes the
    gate (``mk`` supplies a precomputed operand, otherwise it is derived from this call's q and k).  The wide
    gate of 213 is safe only for k-smoothed keys (``diffusers_tpu/kernels/splash.py:596-598``): pass
    ``k_smoothed=True`` when the caller has smoothed them (:func:`smooth_k`, as :func:`sdpa` does); otherwise
    the operand is derived with the halved gate of 106.5, under which no row can flush whatever its mean logit.
    ``qk_fp8`` casts the pre-scaled query and the key to E4M3 and runs the score MMA in 8-bit floats.
    ``block_*``, ``kv_mask_all`` and ``unroll`` are accepted for signature parity and ignored.
    """
    del block_q, block_kv, block_kv_compute, kv_mask_all, unroll
    _check_inputs(query, key, value)
    query, key, value = _dense_last(query), _dense_last(key), _dense_last(value)
    dev = query.device
    if qk_fp8:
        # The reference casts the pre-scaled query and the key to E4M3 in front of the score matmul
        # (diffusers_tpu/kernels/splash.py:420-424, 607-609); P*V stays bf16.
        if use_fixed_m and mk is None:
            raise NotImplementedError("qk_fp8 with use_fixed_m needs a calibrated mk (dtb200.fixed_m.static_fixed_m_operands)")
        if num_splits > 1:
            raise NotImplementedError("qk_fp8 has no split-KV variant")
        s_ = (1.0 / math.sqrt(query.shape[-1])) if scale is None else float(scale)
        query = quantize_e4m3(query, mult=s_ * LOG2_E)
        key = quantize_e4m3(key)
        scale = 1.0 / LOG2_E          # the logits already are in log2 units
    if out is None:
        out = torch.empty(query.shape, dtype=value.dtype, device=dev)
    kv_len_t = _kv_len_tensor(kv_len, query.shape[0], dev)
    flags = _lib.FLAG_QK_FP8 if qk_fp8 else 0
    if zero_padded_rows and kv_len_t is not None:
        flags |= _lib.FLAG_ZERO_PADDED_ROWS
    if use_fixed_m:
        if mk is None:
            mk = fixed_m_operands(query, key, scale=scale,
                                  gate=FIXED_M_SAFE_BOUND if k_smoothed else FIXED_M_RING_SAFE_BOUND)
        flags |= _lib.FLAG_BOUNDED_LOGITS
    else:
        mk = None
    status = _status_buffer(dev)
    p = _fill_params(query, key, value, out, kv_len_t, mk, scale, flags, 1 if qk_fp8 else num_splits, status)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(dev, lib.dtb_attn_workspace_bytes(ctypes.byref(p)))
        st = lib.dtb_attn_fwd(ctypes.byref(p), ws.data_ptr() if ws is not None else None,
                              ws.numel() if ws is not None else 0, _stream_ptr(dev))
    _lib.check(st, "dtb_attn_fwd")
    return out


def describe_launch(batch: int, heads: int, seq_q: int, seq_kv: Optional[int] = None, *, sms: int = 0) -> str:
    """One line saying how the automatic mode launches a call of this shape (the counterpart of the line the reference
    logs per resolved shape, ``diffusers_tpu/kernels/mesh_attention.py:210-214``).  Needs no GPU."""
    p = _lib.AttnParams()
    p.q = p.k = p.v = p.o = 4096          # never dereferenced: the plan depends on the shape alone
    skv = seq_q if seq_kv is None else seq_kv
    p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.D = batch, heads, heads, seq_q, skv, 128
    p.q_stride_s = p.k_stride_s = p.v_stride_s = p.o_stride_s = 128
    p.q_stride_h = p.o_stride_h = seq_q * 128
    p.k_stride_h = p.v_stride_h = skv * 128
    p.q_stride_b = p.o_stride_b = heads * seq_q * 128
    p.k_stride_b = p.v_stride_b = heads * skv * 128
    plan = _lib.LaunchPlan()
    _lib.check(_lib.load().dtb_attn_launch_plan(ctypes.byref(p), int(sms), ctypes.byref(plan)), "dtb_attn_launch_plan")
    n_sms = sms or 148
    head = f"{plan.units} query blocks x {plan.key_tiles} key tiles ({plan.units / n_sms:.2f} waves of {n_sms})"
    if plan.n_pieces == 0:
        return head + ": plain launch, one CTA per query block"
    lens = [plan.tile_end[i] - plan.tile_begin[i] for i in range(plan.n_pieces)]
    return (head + f": {plan.whole_units} whole, the last {plan.tail_units} cut into {plan.n_pieces} pieces of "
            f"{min(lens)}-{max(lens)} key tiles ({plan.n_slots} merged through scratch)")


class ResidualState:
    """Running ``(o, m, l)`` of a ring: ``o`` f32 ``[B,H,Sq,D]`` unnormalised, ``m``/``l`` f32 ``[B,H,Sq]``.

    ``m`` is in log2 units of the scaled logits, so ``lse = m + log2(l)`` is the m-invariant
    quantity the reference's ring merges on (``diffusers_tpu/kernels/splash.py:657-662``).
    """

    def __init__(self, batch: int, heads: int, seq_q: int, device: torch.device):
        self.o = torch.empty(batch, heads, seq_q, 128, dtype=torch.float32, device=device)
        self.m = torch.empty(batch, heads, seq_q, dtype=torch.float32, device=device)
        self.l = torch.empty(batch, heads, seq_q, dtype=torch.float32, device=device)
        self.fresh = True


def residual_attention_(
    state: ResidualState,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    scale: Optional[float] = None,
    use_fixed_m: bool = False,
    mk: Optional[torch.Tensor] = None,
    kv_len: KvLen = None,
    kv_offset: int = 0,
    q_offset: int = 0,
    qk_fp8: bool = False,
) -> ResidualState:
    """Folds one KV shard into ``state`` in place (the fused kernel + merge step of a ring).

    With ``qk_fp8`` the score product runs on E4M3 operands (``diffusers_tpu/kernels/splash.py:420-424``):
    ``query`` and ``key`` may be bf16 (cast here, the query pre-multiplied by ``scale * log2(e)``) or tensors
    already cast with :func:`quantize_e4m3` the same way, which lets a ring cast its query once and move
    one-byte key shards.
    """
    if use_fixed_m and mk is None:
        raise ValueError("use_fixed_m needs the (2, heads) operand mk.")
    if qk_fp8:
        s_ = (1.0 / math.sqrt(query.shape[-1])) if scale is None else float(scale)
        if query.dtype == torch.bfloat16:
            query = quantize_e4m3(query, mult=s_ * LOG2_E)
        if key.dtype == torch.bfloat16:
            key = quantize_e4m3(key)
        if query.dtype != torch.float8_e4m3fn or key.dtype != torch.float8_e4m3fn:
            raise NotImplementedError("qk_fp8 takes bf16 or float8_e4m3fn query and key")
        _check_inputs(value, value, value)
        if query.dim() != 4 or key.shape != value.shape or query.shape[0] != key.shape[0] or query.shape[-1] != 128:
            raise ValueError("query/key/value shapes do not match")
        query, key = query.contiguous(), key.contiguous()
        scale = 1.0 / LOG2_E          # the logits already are in log2 units
    else:
        _check_inputs(query, key, value)
        query, key = _dense_last(query), _dense_last(key)
    value = _dense_last(value)
    dev = query.device
    kv_len_t = _kv_len_tensor(kv_len, query.shape[0], dev)
    flags = (_lib.FLAG_BOUNDED_LOGITS if use_fixed_m else 0) | (_lib.FLAG_QK_FP8 if qk_fp8 else 0)
    p = _fill_params(query, key, value, None, kv_len_t, mk if use_fixed_m else None, scale, flags, 1,
                     _status_buffer(dev))
    r = _lib.AttnResidual(state.o.data_ptr(), state.m.data_ptr(), state.l.data_ptr(), int(kv_offset),
                          int(q_offset), 1 if state.fresh else 0)
    with torch.cuda.device(dev):
        st = _lib.load().dtb_attn_fwd_residual(ctypes.byref(p), ctypes.byref(r), _stream_ptr(dev))
    _lib.check(st, "dtb_attn_fwd_residual")
    state.fresh = False
    return state


def finalize_residual(state: ResidualState, *, dtype: torch.dtype = torch.bfloat16, kv_len: KvLen = None,
                      q_offset: int = 0, zero_padded_rows: bool = True,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``o / l`` cast to bf16: the epilogue of ``splash.py:367-375`` applied to a merged ring state."""
    if dtype != torch.bfloat16:
        raise NotImplementedError("only bfloat16 outputs are supported")
    dev = state.o.device
    B, H, Sq, D = state.o.shape
    if out is None:
        out = torch.empty(B, H, Sq, D, dtype=torch.bfloat16, device=dev)
    kv_len_t = _kv_len_tensor(kv_len, B, dev)
    flags = _lib.FLAG_ZERO_PADDED_ROWS if (zero_padded_rows and kv_len_t is not None) else 0
    p = _lib.AttnParams()
    p.o = out.data_ptr()
    p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.D = B, H, H, Sq, Sq, D
    p.o_stride_b, p.o_stride_h, p.o_stride_s = out.stride()[:3]
    p.kv_len = kv_len_t.data_ptr() if kv_len_t is not None else None
    p.flags = flags
    r = _lib.AttnResidual(state.o.data_ptr(), state.m.data_ptr(), state.l.data_ptr(), 0, int(q_offset), 0)
    with torch.cuda.device(dev):
        st = _lib.load().dtb_attn_finalize(ctypes.byref(p), ctypes.byref(r), _stream_ptr(dev))
    _lib.check(st, "dtb_attn_finalize")
    return out


def residual_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    scale: Optional[float] = None,
    block_q: Optional[int] = None,
    block_kv: Optional[int] = None,
    block_kv_compute: Optional[int] = None,
    use_fixed_m: bool = False,
    qk_fp8: bool = False,
    mk: Optional[torch.Tensor] = None,
    kv_len: KvLen = None,
    kv_offset: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One KV shard's unnormalised ``(o, m, l)``: ``o`` f32 ``[B,H,Sq,D]``, ``m``/``l`` f32 ``[B,H,Sq,1]``.

    Same contract as ``diffusers_tpu/kernels/splash.py:665-742`` (raises ``ValueError`` when
    ``use_fixed_m`` is set without ``mk``, as the reference does at ``:712-713``).
    """
    del block_q, block_kv, block_kv_compute
    if use_fixed_m and mk is None:
        raise ValueError("use_fixed_m needs the (2, heads) operand mk.")
    _check_inputs(query, key, value)
    state = ResidualState(query.shape[0], query.shape[1], query.shape[2], query.device)
    residual_attention_(state, query, key, value, scale=scale, use_fixed_m=use_fixed_m, mk=mk, kv_len=kv_len,
                        kv_offset=kv_offset, qk_fp8=qk_fp8)
    return state.o, state.m.unsqueeze(-1), state.l.unsqueeze(-1)


def sdpa(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    scale: Optional[float] = None,
    enable_gqa: bool = False,
    *,
    kv_len: KvLen = None,
    use_fixed_m: bool = False,
) -> torch.Tensor:
    """SDPA-signature callable, ``[B, H, S, D]`` in and out (``mesh_attention.py:218-261``)."""
    del attn_mask, dropout_p, is_causal, enable_gqa  # Not supported, as in the reference.
    if use_fixed_m:
        # The bounded-logit softmax and k-smoothing go together (mesh_attention.py:234-237): zero-mean keys make
        # every row's largest logit non-negative, which the no-flush guarantee of the 213 gate rests on.
        key = _smooth_k(key, kv_len=kv_len)
        return attention(query, key, value, scale=scale, kv_len=kv_len, use_fixed_m=True, k_smoothed=True)
    return attention(query, key, value, scale=scale, kv_len=kv_len)


def qk_prepass(
    query: torch.Tensor,
    key: torch.Tensor,
    value: Optional[torch.Tensor] = None,
    *,
    q_weight: Optional[torch.Tensor] = None,
    k_weight: Optional[torch.Tensor] = None,
    eps: float = 1e-5,
    rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    kv_len: KvLen = None,
    scale: Optional[float] = None,
    want_mk: bool = False,
    gate: Optional[float] = None,
    smooth_k: bool = False,
):
    """Fused per-head RMSNorm + rotary embedding + pad zeroing + ``(B, S, H, D) -> (B, H, S, D)``.

    ``query, key, value`` are the projections as a DiT block produces them, ``(B, seq, heads, 128)`` bf16
    (any strides with a contiguous last axis); ``rope = (cos, sin)`` are ``(seq, rotary)`` tables that rotate
    the leading ``rotary`` channels and pass the rest through (``apply_rope``,
    ``diffusers_tpu/models/minimax_h3/jax_dit.py:251-262``); the norm is ``x * rsqrt(mean(x^2) + eps) * weight``
    in f32 (``:191-195``); rows at or past ``kv_len[b]`` come out as zeros (``:372-381``).  Returns
    ``(q, k, v, mk)`` laid out ``(B, H, S, D)``; ``mk`` is the ``(2, H)`` bounded-logit operand of the returned
    q and k (``diffusers_tpu/kernels/fixed_m_bound.py:98-118``) when ``want_mk``, else ``None``.
    ``smooth_k`` additionally subtracts the per-head mean key over the valid rows from the returned k
    (``diffusers_tpu/models/minimax_h3/jax_server.py:276-281``); ``mk`` then bounds the smoothed keys.  ``gate``
    defaults to 213 for smoothed keys and to 106.5 otherwise.
    """
    if gate is None:
        gate = FIXED_M_SAFE_BOUND if smooth_k else FIXED_M_RING_SAFE_BOUND
    tensors = [query, key] + ([value] if value is not None else [])
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("qk_prepass needs CUDA tensors: dtb200 has no CPU path")
        if t.dtype != torch.bfloat16 or t.dim() != 4 or t.shape[-1] != 128:
            raise NotImplementedError(f"expected bf16 (B, S, H, 128), got {t.dtype} {tuple(t.shape)}")
        if t.shape != query.shape:
            raise ValueError("query, key and value must have the same shape")
    tensors = [t if (t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3]))
               else t.contiguous() for t in tensors]
    B, S, H, Dh = query.shape
    dev = query.device
    outs = [torch.empty(B, H, S, Dh, dtype=torch.bfloat16, device=dev) for _ in tensors]
    p = _lib.PrepassParams()
    p.q_in, p.k_in = tensors[0].data_ptr(), tensors[1].data_ptr()
    p.q_out, p.k_out = outs[0].data_ptr(), outs[1].data_ptr()
    for name, t in zip(("q", "k", "v"), tensors):
        arr = getattr(p, name + "_strides")
        arr[0], arr[1], arr[2] = t.stride()[:3]
    if value is not None:
        p.v_in, p.v_out = tensors[2].data_ptr(), outs[2].data_ptr()
    keep = []
    for name, wt in (("q_weight", q_weight), ("k_weight", k_weight)):
        if wt is not None:
            wt = wt.to(device=dev, dtype=torch.float32).contiguous()
            if wt.numel() != Dh:
                raise ValueError(f"{name} must have {Dh} entries")
            keep.append(wt)
            setattr(p, name, wt.data_ptr())
    if rope is not None:
        cos, sin = (t.to(device=dev, dtype=torch.float32).contiguous() for t in rope)
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[0] != S:
            raise ValueError(f"rope tables must both be (seq={S}, rotary), got {tuple(cos.shape)} and {tuple(sin.shape)}")
        keep += [cos, sin]
        p.cos, p.sin, p.rotary = cos.data_ptr(), sin.data_ptr(), cos.shape[1]
    kv_len_t = _kv_len_tensor(kv_len, B, dev)
    p.kv_len = kv_len_t.data_ptr() if kv_len_t is not None else None
    mk = None
    if want_mk:
        norms = torch.empty(2 * H, dtype=torch.float32, device=dev)
        mk = torch.empty(2, H, dtype=torch.float32, device=dev)
        keep.append(norms)
        p.norms, p.mk_out = norms.data_ptr(), mk.data_ptr()
    p.eps, p.scale, p.gate = float(eps), float(scale) if scale is not None else 0.0, float(gate)
    p.B, p.S, p.H, p.D = B, S, H, Dh
    with torch.cuda.device(dev):
        st = _lib.load().dtb_qk_prepass(ctypes.byref(p), _stream_ptr(dev))
    _lib.check(st, "dtb_qk_prepass")
    if smooth_k:
        # second pass over k only: the mean is a property of the finished (normed, rotated) keys
        _, k_norms = _smooth_k(outs[1], kv_len=kv_len_t, out=outs[1], want_norms=True)
        if want_mk:
            with torch.cuda.device(dev):
                st = _lib.load().dtb_fixed_m_from_norms(norms.data_ptr(), k_norms.data_ptr(), H, H, float(gate),
                                                        mk.data_ptr(), _stream_ptr(dev))
            _lib.check(st, "dtb_fixed_m_from_norms")
    return outs[0], outs[1], (outs[2] if value is not None else None), mk


def _out_proj_params(o: torch.Tensor, w: torch.Tensor) -> _lib.OutProjParams:
    if not o.is_cuda or not w.is_cuda:
        raise RuntimeError("out_proj needs CUDA tensors: dtb200 has no CPU path")
    if o.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise NotImplementedError("out_proj takes bfloat16 operands")
    if o.dim() != 4 or o.shape[-1] != 128:
        raise NotImplementedError(f"attention output must be [B, heads, seq, 128], got {tuple(o.shape)}")
    if w.dim() != 2 or w.shape[0] != o.shape[1] * 128 or w.shape[1] % 8:
        raise ValueError(f"weight must be [heads * 128 = {o.shape[1] * 128}, N] with N a multiple of 8, got {tuple(w.shape)}")
    p = _lib.OutProjParams()
    p.o = o.data_ptr()
    p.o_stride_b, p.o_stride_h, p.o_stride_s = o.stride()[:3]
    p.w, p.w_stride_k = w.data_ptr(), w.stride(0)
    p.B, p.H_local, p.S, p.D, p.N = o.shape[0], o.shape[1], o.shape[2], 128, w.shape[1]
    p.status = _status_buffer(o.device).data_ptr()
    return p


def out_proj(o: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[b, s, :] = sum_h o[b, h, s, :] @ w[h*128:(h+1)*128, :]``: the ``to_out`` projection applied to the
    attention output in its ``[B, heads, seq, 128]`` layout (no heads -> channels transpose), bf16 ``[B, seq, N]``.

    With head-sharded attention output (``diffusers_tpu/models/minimax_h3/jax_image_pipeline.py:574-593``) ``w`` holds
    the rows of the weight that belong to the local heads and the result is this GPU's partial sum; see
    :func:`out_proj_reduce_` for the form that adds it straight into the owners' buffers."""
    o, w = _dense_last(o), (w if (w.stride(1) == 1 and w.data_ptr() % 16 == 0 and w.stride(0) % 8 == 0) else w.contiguous())
    p = _out_proj_params(o, w)
    if out is None:
        out = torch.empty(o.shape[0], o.shape[2], w.shape[1], dtype=torch.bfloat16, device=o.device)
    p.out = out.data_ptr()
    p.out_stride_b, p.out_stride_s = out.stride()[:2]
    p.n_dest = 0
    with torch.cuda.device(o.device):
        st = _lib.load().dtb_out_proj(ctypes.byref(p), _stream_ptr(o.device))
    _lib.check(st, "dtb_out_proj")
    return out


def out_proj_reduce_(o: torch.Tensor, w: torch.Tensor, dest_ptrs: Sequence[int], rows_per_dest: int, *,
                     partials_from: Optional[int] = None) -> None:
    """Sends this GPU's partial projection to the buffers that own the rows: row ``b * seq + s`` of the flattened
    result goes to ``dest_ptrs[row // rows_per_dest]``, given by its device address (this GPU's or a peer's mapped
    into this process).

    ``partials_from=r``: bf16 rows stored into slot ``r`` of the destination's staging buffer, bf16
    ``[n_src, rows_per_dest, N]``, for :func:`sum_partials` on the owner.  ``partials_from=None``: f32 sums added by
    vector reductions into the destination's f32 ``[rows_per_dest, N]`` buffer, which must already hold what they are
    added to (zeros, a bias, the residual).  The caller orders the ranks around the call."""
    o, w = _dense_last(o), (w if (w.stride(1) == 1 and w.data_ptr() % 16 == 0 and w.stride(0) % 8 == 0) else w.contiguous())
    p = _out_proj_params(o, w)
    if not 1 <= len(dest_ptrs) <= 8:
        raise ValueError("1 to 8 destination buffers")
    for i, ptr in enumerate(dest_ptrs):
        p.red_dst[i] = int(ptr)
    p.n_dest, p.rows_per_dest = len(dest_ptrs), int(rows_per_dest)
    if partials_from is not None:
        p.partials, p.src_rank = 1, int(partials_from)
    with torch.cuda.device(o.device):
        st = _lib.load().dtb_out_proj(ctypes.byref(p), _stream_ptr(o.device))
    _lib.check(st, "dtb_out_proj")


def sum_partials(staged: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 ``[rows, N]`` sum (f32 accumulation, slot order) of the staged partial projections ``[n_src, rows, N]``."""
    if not staged.is_cuda or staged.dtype != torch.bfloat16 or staged.dim() != 3 or not staged.is_contiguous():
        raise NotImplementedError("sum_partials takes a contiguous CUDA bf16 [n_src, rows, N] tensor")
    n_src, rows, N = staged.shape
    if out is None:
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=staged.device)
    with torch.cuda.device(staged.device):
        st = _lib.load().dtb_sum_partials(staged.data_ptr(), n_src, rows, N, out.data_ptr(), _stream_ptr(staged.device))
    _lib.check(st, "dtb_sum_partials")
    return out


class BlockTable:
    """Device-resident block-sparsity table at the kernel's granularity (256 query rows x 128 keys).

    Built once per layout with :func:`make_block_table` and passed to :func:`sparse_attention`.
    """

    def __init__(self, table: torch.Tensor, count: torch.Tensor, head_class: Optional[torch.Tensor], seq_q: int):
        self.table, self.count, self.head_class, self.seq_q = table, count, head_class, seq_q
        self.n_classes, self.q_blocks, self.width = table.shape


def make_block_table(kv_table, *, seq_q: int, seq_kv: int, block_q: int, block_kv: int, device="cuda",
                     heads: Optional[int] = None) -> BlockTable:
    """Converts a reference-style table to the kernel's granularity and uploads it.

    ``kv_table`` is what ``diffusers_tpu/kernels/sparse_splash.py:568-649`` takes: per query block of ``block_q``
    rows the sorted list of key blocks (of ``block_kv`` keys) to visit, shared by all heads; or
    ``(classes, head_class)`` with one such table per head class and a class index per head.  ``block_q`` must be a
    multiple of 256 and ``block_kv`` a multiple of 128 (the kernel's tile), so that a reference block is a whole
    number of kernel tiles; the result visits exactly the same (query, key) pairs.
    """
    if block_q % 256 or block_kv % 128:
        raise NotImplementedError("block_q must be a multiple of 256 and block_kv a multiple of 128")
    if isinstance(kv_table, tuple):
        classes, head_class = kv_table
        head_class = torch.as_tensor(list(head_class), dtype=torch.int32)
        if heads is not None and head_class.numel() != heads:
            raise ValueError("head_class must have one entry per head")
    else:
        classes, head_class = [kv_table], None
    qb_ratio, kb_ratio = block_q // 256, block_kv // 128
    n_q = (seq_q + 255) // 256
    n_kv_tiles = (seq_kv + 127) // 128
    rows = []
    for table in classes:
        if len(table) != (seq_q + block_q - 1) // block_q:
            raise ValueError(f"table has {len(table)} query blocks, expected {(seq_q + block_q - 1) // block_q}")
        per_q = []
        for qb in range(n_q):
            blocks = sorted(set(int(x) for x in table[qb // qb_ratio]))
            tiles = [b * kb_ratio + i for b in blocks for i in range(kb_ratio) if b * kb_ratio + i < n_kv_tiles]
            per_q.append(tiles)
        rows.append(per_q)
    width = max(1, max(len(t) for per_q in rows for t in per_q))
    tab = torch.zeros(len(rows), n_q, width, dtype=torch.int32)
    cnt = torch.zeros(len(rows), n_q, dtype=torch.int32)
    for c, per_q in enumerate(rows):
        for qb, tiles in enumerate(per_q):
            cnt[c, qb] = len(tiles)
            if tiles:
                tab[c, qb, :len(tiles)] = torch.tensor(tiles, dtype=torch.int32)
    return BlockTable(tab.to(device), cnt.to(device), head_class.to(device) if head_class is not None else None, seq_q)


def sparse_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    kv_table: BlockTable,
    scale: Optional[float] = None,
    kv_len: KvLen = None,
    use_fixed_m: bool = False,
    mk: Optional[torch.Tensor] = None,
    zero_padded_rows: bool = True,
    out: Optional[torch.Tensor] = None,
    k_smoothed: bool = False,
) -> torch.Tensor:
    """Block-sparse joint attention: each query block attends only to the key tiles its table row lists.

    Same contract as ``attention`` otherwise (``diffusers_tpu/kernels/sparse_splash.py:568-649``); a table that
    lists every tile gives the dense result bit for bit.  Query blocks with an empty row come back as zeros.
    """
    _check_inputs(query, key, value)
    query, key, value = _dense_last(query), _dense_last(key), _dense_last(value)
    if kv_table.seq_q != query.shape[2]:
        raise ValueError(f"table was built for seq_q={kv_table.seq_q}, got {query.shape[2]}")
    if kv_table.head_class is not None and kv_table.head_class.numel() != query.shape[1]:
        raise ValueError("table head classes do not match the number of heads")
    dev = query.device
    if out is None:
        out = torch.empty(query.shape, dtype=query.dtype, device=dev)
    kv_len_t = _kv_len_tensor(kv_len, query.shape[0], dev)
    flags = _lib.FLAG_ZERO_PADDED_ROWS if (zero_padded_rows and kv_len_t is not None) else 0
    if use_fixed_m:
        if mk is None:
            mk = fixed_m_operands(query, key, scale=scale,
                                  gate=FIXED_M_SAFE_BOUND if k_smoothed else FIXED_M_RING_SAFE_BOUND)
        flags |= _lib.FLAG_BOUNDED_LOGITS
    else:
        mk = None
    p = _fill_params(query, key, value, out, kv_len_t, mk, scale, flags, 1, _status_buffer(dev))
    tb = _lib.BlockTable(kv_table.table.data_ptr(), kv_table.count.data_ptr(),
                         kv_table.head_class.data_ptr() if kv_table.head_class is not None else None,
                         kv_table.n_classes, kv_table.q_blocks, kv_table.width)
    with torch.cuda.device(dev):
        st = _lib.load().dtb_attn_fwd_sparse(ctypes.byref(p), ctypes.byref(tb), _stream_ptr(dev))
    _lib.check(st, "dtb_attn_fwd_sparse")
    return out
