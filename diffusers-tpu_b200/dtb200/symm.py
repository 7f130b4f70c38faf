"""Peer-memory versions of the multi-GPU placements: this library's own kernels move the data over NVLink.

Buffers that other ranks write to or read from live in one symmetric-memory arena per process group
(``torch.distributed._symmetric_memory``: the same allocation on every rank, each mapped into every
process), so a kernel on one GPU can address its peers' buffers with plain loads and stores.

* :class:`UlyssesP2P` — sequence-sharded in, sequence-sharded out.  One ``scatter_heads`` kernel writes this
  rank's q, k and v head groups straight into the owners' ``[B, H/P, S, D]`` buffers (the first all-to-all of
  ``diffusers_tpu/backends/qwen21_core_tt.py:108-115`` without send/receive staging or layout copies), and the
  attention kernel's epilogue stores every output row into the buffer of the rank that owns that part of the
  sequence (the second all-to-all, ``:116-121``, fused into the kernel).  Two cross-rank barriers remain.
* :class:`RingPull` — ring-KV without forwarding: every rank publishes its K/V shard once, and each step's
  shard is pulled from its owner by the copy engines into a local double buffer while the previous shard
  is being folded by the residual kernel (``diffusers_tpu/kernels/splash.py:657-662`` gives the merge rule).

No TMA load, multicast or otherwise, ever targets peer memory here: remote K/V are copied to local HBM
first, and remote writes are plain 16-byte stores.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib, ops

D = 128


class SymmArena:
    """One symmetric allocation carved into named regions; every region exists on every rank of ``group``."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (nbytes + 255) // 256 * 256
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs = list(self.handle.buffer_ptrs)
        self._cursor = 0

    def carve(self, nbytes: int) -> int:
        off = self._cursor
        self._cursor = (off + nbytes + 255) // 256 * 256
        if self._cursor > self.nbytes:
            raise RuntimeError("symmetric arena exhausted")
        return off

    def local(self, offset: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty((), dtype=dtype).element_size()
        return self.buf[offset:offset + n * esz].view(dtype).view(*shape)

    def peer(self, rank: int, offset: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        if esz == 1:     # one-byte types are mapped as bytes and reinterpreted
            return self.handle.get_buffer(rank, tuple(shape), torch.uint8, offset).view(dtype)
        return self.handle.get_buffer(rank, tuple(shape), dtype, offset // esz)

    def ptr(self, rank: int, offset: int) -> int:
        return self.ptrs[rank] + offset

    def barrier(self, channel: int = 0) -> None:
        """Stream-ordered barrier over the group (a kernel on the current stream)."""
        self.handle.barrier(channel=channel)


class UlyssesP2P:
    """Head-parallel attention on a sequence-sharded stream with both exchanges done by peer stores."""

    def __init__(self, batch: int, heads: int, seq_local: int, group=None, device: Optional[torch.device] = None):
        P = dist.get_world_size(group)
        if heads % P:
            raise ValueError(f"{heads} heads do not divide over {P} ranks")
        if P > 8:
            raise ValueError("at most 8 peers")
        self.B, self.H, self.Sl, self.P = batch, heads, seq_local, P
        self.Hl, self.S = heads // P, seq_local * P
        y_bytes = batch * self.Hl * self.S * D * 2
        o_bytes = batch * heads * seq_local * D * 2
        self.arena = SymmArena(3 * y_bytes + o_bytes + 4096, group, device)
        self.rank = self.arena.rank
        self.y_off = [self.arena.carve(y_bytes) for _ in range(3)]
        self.o_off = self.arena.carve(o_bytes)
        self.y = [self.arena.local(off, (batch, self.Hl, self.S, D)) for off in self.y_off]
        self.out = self.arena.local(self.o_off, (batch, heads, seq_local, D))

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, kv_len=None,
                 scale: Optional[float] = None) -> torch.Tensor:
        """``q, k, v``: this rank's ``[B, H, S/P, D]`` shards; returns its ``[B, H, S/P, D]`` output shard.

        The returned tensor is a view of the arena and is overwritten by the next call."""
        dev = self.arena.device
        lib = _lib.load()
        stream = torch.cuda.current_stream(dev).cuda_stream
        srcs = [ops._dense_last(t) for t in (q, k, v)]
        for t in srcs:
            if tuple(t.shape) != (self.B, self.H, self.Sl, D) or t.dtype != torch.bfloat16:
                raise ValueError(f"expected bf16 {(self.B, self.H, self.Sl, D)}, got {t.dtype} {tuple(t.shape)}")
        sp = _lib.ScatterHeadsParams()
        for i, t in enumerate(srcs):
            sp.src[i] = t.data_ptr()
            sp.stride_b[i], sp.stride_h[i], sp.stride_s[i] = t.stride()[:3]
            for r in range(self.P):
                sp.dst[i][r] = self.arena.ptr(r, self.y_off[i])
        sp.n_tensors, sp.n_peers, sp.rank = 3, self.P, self.rank
        sp.B, sp.H, sp.S_local, sp.D = self.B, self.H, self.Sl, D
        with torch.cuda.device(dev):
            _lib.check(lib.dtb_scatter_heads(ctypes.byref(sp), stream), "dtb_scatter_heads")
            self.arena.barrier(0)   # every rank's head groups have landed here
            yq, yk, yv = self.y
            kv_len_t = ops._kv_len_tensor(kv_len, self.B, dev)
            flags = _lib.FLAG_ZERO_PADDED_ROWS if kv_len_t is not None else 0
            p = ops._fill_params(yq, yk, yv, None, kv_len_t, None, scale, flags, 0, ops._status_buffer(dev))
            sc = _lib.AttnScatter()
            ws = ops._workspace(dev, lib.dtb_attn_workspace_bytes(ctypes.byref(p)))   # lets the last wave be balanced
            if ws is not None:
                sc.workspace, sc.workspace_bytes = ws.data_ptr(), ws.numel()
            for r in range(self.P):
                sc.out_ptrs[r] = self.arena.ptr(r, self.o_off)
            sc.n_peers, sc.shard_rows = self.P, self.Sl
            sc.head_offset, sc.total_heads = self.rank * self.Hl, self.H
            _lib.check(lib.dtb_attn_fwd_scatter(ctypes.byref(p), ctypes.byref(sc), stream), "dtb_attn_fwd_scatter")
            self.arena.barrier(1)   # every rank's rows of my shard have landed, and nobody still reads y
        return self.out


class RingPull:
    """Ring-KV attention where each step's K/V shard is pulled from its owner by the copy engines.

    ``qk_fp8`` moves and multiplies E4M3 keys (half the bytes per K shard) and casts the pre-scaled query once
    per call; with ``use_fixed_m`` every step runs the bounded-logit softmax with one operand for the whole ring
    (``diffusers_tpu/kernels/fixed_m_bound.py:121-155``: the same ``m`` for all heads, the gate halved because
    ring shards are not k-smoothed) — the reference's fastest ring configuration (``:313-316``).
    """

    def __init__(self, batch: int, heads: int, seq_local: int, group=None, device: Optional[torch.device] = None,
                 qk_fp8: bool = False):
        self.P = dist.get_world_size(group)
        self.group = group
        self.B, self.H, self.Sl = batch, heads, seq_local
        self.qk_fp8 = qk_fp8
        self.k_dtype = torch.float8_e4m3fn if qk_fp8 else torch.bfloat16
        v_shard = batch * heads * seq_local * D * 2
        k_shard = v_shard // 2 if qk_fp8 else v_shard
        self.arena = SymmArena(k_shard + v_shard + 4096, group, device)
        self.rank = self.arena.rank
        self.k_off, self.v_off = self.arena.carve(k_shard), self.arena.carve(v_shard)
        shape = (batch, heads, seq_local, D)
        dev = self.arena.device
        self.k_pub = self.arena.local(self.k_off, shape, self.k_dtype)
        self.v_pub = self.arena.local(self.v_off, shape)
        self.bufs = [(torch.empty(shape, dtype=self.k_dtype, device=dev),
                      torch.empty(shape, dtype=torch.bfloat16, device=dev)) for _ in range(2)] if self.P > 1 else []
        self.copy_stream = torch.cuda.Stream(dev)
        self.ready = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]
        self.state = ops.ResidualState(batch, heads, seq_local, dev)
        self.shape = shape

    def schedule(self) -> List[int]:
        return [(self.rank - t) % self.P for t in range(self.P)]

    def ring_operand(self, q: torch.Tensor, k: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
        """The ``(2, heads)`` bounded-logit operand of a whole ring: per-head row-norm maxima of this rank's shards,
        reduced with MAX over the ranks, then ``fixed_m.ring_fixed_m_operands``.  Callers with calibrated norms
        (``fixed_m.static_fixed_m_operands``) pass their own ``mk`` instead and skip this pass."""
        from . import fixed_m

        qn, kn = ops.row_norm_maxima(q, k, scale=scale)
        if self.P > 1:
            both = torch.cat([qn, kn])
            dist.all_reduce(both, op=dist.ReduceOp.MAX, group=self.group)
            qn, kn = both[:qn.numel()], both[qn.numel():]
        if kn.numel() != qn.numel():
            kn = kn.repeat_interleave(qn.numel() // kn.numel())
        if self.qk_fp8:
            qn = qn * (1.0 + 2.0 ** -4)      # E4M3 rounding can raise a magnitude by 2^-4, on q and on k (:293-297)
            kn = kn * (1.0 + 2.0 ** -4)
        return fixed_m.ring_fixed_m_operands(qn, kn)

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, kv_len=None, scale: Optional[float] = None,
                 out: Optional[torch.Tensor] = None, zero_padded_rows: bool = True, use_fixed_m: bool = False,
                 mk: Optional[torch.Tensor] = None) -> torch.Tensor:
        dev = self.arena.device
        main = torch.cuda.current_stream(dev)
        Sl = self.Sl
        sched = self.schedule()
        if use_fixed_m and mk is None:
            mk = self.ring_operand(q, k, scale)
        if self.qk_fp8:
            import math

            s_ = (1.0 / math.sqrt(D)) if scale is None else float(scale)
            q = ops.quantize_e4m3(q, mult=s_ * ops.LOG2_E)
            k = ops.quantize_e4m3(k)
        if self.P > 1:
            self.k_pub.copy_(k)
            self.v_pub.copy_(v)
            self.arena.barrier(0)        # every shard is published
            for ev in self.consumed:
                ev.record(main)
        self.state.fresh = True
        k_cur, v_cur = k, v
        for t, origin in enumerate(sched):
            if t + 1 < self.P:
                nxt = sched[t + 1]
                kb, vb = self.bufs[t % 2]
                with torch.cuda.stream(self.copy_stream):
                    if t == 0:
                        self.copy_stream.wait_stream(main)       # after the barrier
                    self.copy_stream.wait_event(self.consumed[t % 2])
                    kb.copy_(self.arena.peer(nxt, self.k_off, self.shape, self.k_dtype), non_blocking=True)
                    vb.copy_(self.arena.peer(nxt, self.v_off, self.shape), non_blocking=True)
                    self.ready[t % 2].record(self.copy_stream)
            ops.residual_attention_(self.state, q, k_cur, v_cur, scale=scale, kv_len=kv_len, kv_offset=origin * Sl,
                                    q_offset=self.rank * Sl, use_fixed_m=use_fixed_m, mk=mk, qk_fp8=self.qk_fp8)
            if t >= 1:
                self.consumed[(t - 1) % 2].record(main)          # the buffer step t read may be refilled
            if t + 1 < self.P:
                main.wait_event(self.ready[t % 2])
                k_cur, v_cur = self.bufs[t % 2]
        res = ops.finalize_residual(self.state, kv_len=kv_len, q_offset=self.rank * Sl,
                                    zero_padded_rows=zero_padded_rows, out=out)
        if self.P > 1:
            self.arena.barrier(1)        # nobody still pulls from a shard that the next call republishes
        return res


class OutProjReduceScatter:
    """``to_out`` behind head-sharded attention output, with the reduce-scatter over the head shards done by the GEMM.

    Every rank multiplies its own heads' attention output ``[B, H/P, S, 128]`` (read in place, no transpose) by its rows
    of the projection weight and sends each finished tile straight to the rank that owns those rows, so the transfer
    over NVLink runs under the GEMM.  This is the all-reduce that follows keep-heads attention in
    ``diffusers_tpu/models/minimax_h3/jax_image_pipeline.py:574-593`` up to its all-gather half: each rank ends up
    with rows ``[rank * B*S/P, (rank + 1) * B*S/P)`` of the projected stream.

    ``exact=False`` (default): bf16 partial rows stored into the owner's staging slot for the sending rank, summed
    there in f32 - the same bytes on the wire as a bf16 reduce-scatter; returns bf16.  ``exact=True``: f32 partial sums
    added into the owner's shard by vector reductions (twice the bytes, atomics over NVLink); returns f32.
    """

    def __init__(self, batch: int, seq: int, n_out: int, group=None, device: Optional[torch.device] = None,
                 exact: bool = False):
        self.P = dist.get_world_size(group)
        if self.P > 8:
            raise ValueError("at most 8 peers")
        rows = batch * seq
        if rows % self.P:
            raise ValueError(f"{rows} rows do not divide over {self.P} ranks")
        self.B, self.S, self.N, self.rows, self.exact = batch, seq, n_out, rows // self.P, exact
        nbytes = self.rows * n_out * (4 if exact else 2 * self.P)
        self.arena = SymmArena(nbytes + 4096, group, device)
        self.rank = self.arena.rank
        self.off = self.arena.carve(nbytes)
        if exact:
            self.acc = self.arena.local(self.off, (self.rows, n_out), torch.float32)
        else:
            self.staged = self.arena.local(self.off, (self.P, self.rows, n_out), torch.bfloat16)
            self.result = torch.empty(self.rows, n_out, dtype=torch.bfloat16, device=self.arena.device)

    def __call__(self, o_local: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
        """Returns this rank's ``[B*S/P, N]`` row shard of the summed projection (overwritten by the next call)."""
        dev = self.arena.device
        if tuple(o_local.shape[::2]) != (self.B, self.S) or w_local.shape[1] != self.N:
            raise ValueError("shapes do not match the buffers this object was built for")
        ptrs = [self.arena.ptr(r, self.off) for r in range(self.P)]
        with torch.cuda.device(dev):
            if self.exact:
                self.acc.zero_()
                self.arena.barrier(0)        # every shard is zero before anybody adds to it
                ops.out_proj_reduce_(o_local, w_local, ptrs, self.rows)
                self.arena.barrier(1)        # every rank's contributions to my shard have landed
                return self.acc
            self.arena.barrier(0)            # every owner has summed the previous call's slots
            ops.out_proj_reduce_(o_local, w_local, ptrs, self.rows, partials_from=self.rank)
            self.arena.barrier(1)            # every rank's rows of my shard have landed
            return ops.sum_partials(self.staged, out=self.result)
