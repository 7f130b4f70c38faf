"""Run under torchrun on N GPUs: checks a multi-GPU driver against the CPU oracle on sampled rows.

    python -m torch.distributed.run --nproc-per-node N tests/multi_gpu_check.py MODE [S] [H] [B]

MODE: ulysses | ring (NCCL collectives), ulysses-p2p | ring-pull (this library's peer-memory kernels),
ring-pull-fixed-m (bounded-logit softmax with the ring operand), ring-pull-fp8 (E4M3 q/k + that operand),
out-proj / out-proj-exact (the projection behind head-sharded attention output with its reduce-scatter fused into
the GEMM: bf16 partial rows stored to the owners and summed there / f32 reductions into the owners' shards).
Inputs are generated shard by shard on the GPUs (no rank ever builds the whole tensor on the host); for the
check every rank gathers the keys and values of two heads and compares a strided sample of its own query rows,
plus its last rows, with the fp32 oracle.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "diffusers-tpu_b200"))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import dtb200  # noqa: E402
from dtb200 import parallel  # noqa: E402
from oracle import attn_oracle as O  # noqa: E402

CHECK_HEADS = 2
SAMPLE_ROWS = 96
TAIL_ROWS = 32


def make_shard(B, H, Sl, rank, dev):
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q = torch.randn(B, H, Sl, 128, generator=g, device=dev)
    k = torch.randn(B, H, Sl, 128, generator=g, device=dev)
    v = torch.randn(B, H, Sl, 128, generator=g, device=dev)
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True)) * 2).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    return q, k, v.to(torch.bfloat16)


def check_out_proj(mode, S, H, B, rank, world, dev):
    """Every rank holds H / world heads of an attention output and the matching rows of a [H * 128, H * 128] weight;
    the fused GEMM + reduce-scatter must leave on each rank its row shard of the full projection (f32)."""
    from dtb200 import symm

    Hl, N = H // world, H * 128
    g = torch.Generator(device=dev).manual_seed(77 + rank)
    o_local = torch.randn(B, Hl, S, 128, generator=g, device=dev).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(5)
    w = (torch.randn(H * 128, N, generator=gw, device=dev) * (H * 128) ** -0.5).to(torch.bfloat16)
    exact = mode == "out-proj-exact"
    op = symm.OutProjReduceScatter(B, S, N, device=dev, exact=exact)
    for _ in range(2):      # twice: the buffers are reused
        got = op(o_local, w[rank * Hl * 128:(rank + 1) * Hl * 128]).clone().float()
    dtb200.check_device_status(dev)
    parts = [torch.empty_like(o_local) for _ in range(world)]
    dist.all_gather(parts, o_local)
    o_all = torch.cat(parts, dim=1)
    rows = B * S // world
    ref = O.out_proj(o_all, w).reshape(B * S, N)[rank * rows:(rank + 1) * rows]
    err = (got.cpu() - ref).abs()
    scale = max(1.0, ref.abs().max().item())
    # exact: f32 sums of f32 partials; default: bf16 partial rows (one rounding per contributing rank) and a bf16 result
    tol = 1e-3 * scale if exact else (world + 1) * 2.0 ** -8 * scale
    ok = torch.tensor([float(err.max().item() <= tol)], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    print(f"rank {rank}: out-proj S={S} H={H} B={B} max_abs={err.max().item():.3e} (row scale {scale:.2f})", flush=True)
    if rank == 0:
        print("PARITY OK" if ok.item() == 1.0 else "PARITY FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() == 1.0 else 1)


def main():
    mode = sys.argv[1]
    S = int(sys.argv[2]) if len(sys.argv) > 2 else 2048
    H = int(sys.argv[3]) if len(sys.argv) > 3 else 8
    B = int(sys.argv[4]) if len(sys.argv) > 4 else 2
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if mode in ("out-proj", "out-proj-exact"):
        return check_out_proj(mode, S, H, B, rank, world, dev)
    assert S % world == 0, "the sequence must divide over the ranks"
    Sl = S // world
    q, k, v = make_shard(B, H, Sl, rank, dev)
    kv_len = torch.tensor([S - 17 * (b + 1) for b in range(B)], dtype=torch.int32)
    fp8 = mode == "ring-pull-fp8"
    if mode in ("ulysses", "ring"):
        fn = parallel.ulysses_attention if mode == "ulysses" else parallel.ring_attention
        out = fn(q, k, v, kv_len=kv_len.to(dev))
    else:
        from dtb200 import symm

        if mode == "ulysses-p2p":
            op, kw = symm.UlyssesP2P(B, H, Sl, device=dev), {}
        else:
            op = symm.RingPull(B, H, Sl, device=dev, qk_fp8=fp8)
            kw = {"use_fixed_m": mode != "ring-pull"}
        for _ in range(2):      # twice: buffers are reused across calls
            out = op(q, k, v, kv_len=kv_len.to(dev), **kw).clone()
    dtb200.check_device_status(dev)

    # oracle on the first CHECK_HEADS heads: whole keys and values gathered, a sample of this rank's query rows
    hs = min(CHECK_HEADS, H)
    parts_k = [torch.empty(B, hs, Sl, 128, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    parts_v = [torch.empty_like(parts_k[0]) for _ in range(world)]
    dist.all_gather(parts_k, k[:, :hs].contiguous())
    dist.all_gather(parts_v, v[:, :hs].contiguous())
    k_all, v_all = torch.cat(parts_k, dim=2), torch.cat(parts_v, dim=2)
    local_rows = torch.cat([torch.arange(0, Sl, max(1, Sl // SAMPLE_ROWS)), torch.arange(max(Sl - TAIL_ROWS, 0), Sl)]).unique()
    q_s = q[:, :hs, local_rows.to(dev)]
    scale = None
    if fp8:   # the variant is compared on the operands it multiplies (E4M3 q * scale * log2e and k)
        c = (128 ** -0.5) * O.LOG2_E
        q_s = dtb200.quantize_e4m3(q_s.contiguous(), mult=c).float()
        k_all = dtb200.quantize_e4m3(k_all).float()
        scale = 1.0 / O.LOG2_E
    ref = O.attention_fp32(q_s, k_all, v_all, kv_len=kv_len, scale=scale, zero_padded_rows=False)
    global_rows = local_rows + rank * Sl
    for b in range(B):
        ref[b, :, global_rows >= int(kv_len[b])] = 0
    err = (out[:, :hs, local_rows.to(dev)].float().cpu() - ref).abs()
    ok = torch.tensor([float(err.max() <= 2e-2 and err.mean() <= 2e-3)], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    print(f"rank {rank}: {mode} S={S} H={H} B={B} rows={len(local_rows)} max_abs={err.max().item():.3e} "
          f"mean_abs={err.mean().item():.3e}", flush=True)
    if rank == 0:
        print("PARITY OK" if ok.item() == 1.0 else "PARITY FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
