"""Run under torchrun on N GPUs: checks a multi-GPU driver against the CPU oracle on sampled rows.

    python -m torch.distributed.run --nproc-per-node N tests/multi_gpu_check.py {ulysses|ring|ulysses-p2p|ring-pull} [S] [H] [B]
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


def main():
    mode = sys.argv[1]
    S = int(sys.argv[2]) if len(sys.argv) > 2 else 2048
    H = int(sys.argv[3]) if len(sys.argv) > 3 else 8
    B = int(sys.argv[4]) if len(sys.argv) > 4 else 2
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(123)
    q, k, v = (torch.randn(B, H, S, 128, generator=g) for _ in range(3))
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True)) * 2).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    v = v.to(torch.bfloat16)
    kv_len = torch.tensor([S - 17 * (b + 1) for b in range(B)], dtype=torch.int32)
    Sl = S // world
    sl = slice(rank * Sl, (rank + 1) * Sl)
    shard = [t[:, :, sl].contiguous().to(dev) for t in (q, k, v)]
    if mode in ("ulysses", "ring"):
        fn = parallel.ulysses_attention if mode == "ulysses" else parallel.ring_attention
        out = fn(*shard, kv_len=kv_len.to(dev))
    else:
        from dtb200 import symm

        cls = symm.UlyssesP2P if mode == "ulysses-p2p" else symm.RingPull
        op = cls(B, H, Sl, device=dev)
        for _ in range(2):      # twice: buffers are reused across calls
            out = op(*shard, kv_len=kv_len.to(dev)).clone()
    dtb200.check_device_status(dev)
    rows = torch.arange(rank * Sl, (rank + 1) * Sl, max(1, Sl // 64))
    ref = O.attention_fp32(q, k, v, kv_len=kv_len, rows=rows)
    err = (out[:, :, (rows - rank * Sl).to(dev)].float().cpu() - ref).abs()
    ok = torch.tensor([float(err.max() <= 2e-2 and err.mean() <= 2e-3)], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    print(f"rank {rank}: max_abs={err.max().item():.3e} mean_abs={err.mean().item():.3e}", flush=True)
    if rank == 0:
        print("PARITY OK" if ok.item() == 1.0 else "PARITY FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
