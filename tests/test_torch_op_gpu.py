"""The torch custom op and the multi-GPU drivers on real devices."""
import os
import subprocess
import sys

import pytest
import torch

import dtb200
from dtb200 import torch_op
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rand(B, H, S, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, H, S, 128, generator=g) for _ in range(3))
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    return q, k, v.to(torch.bfloat16)


def test_custom_op_matches_oracle_and_traces():
    q, k, v = _rand(2, 2, 1280, 1)
    kv_len = torch.tensor([1280, 1000], dtype=torch.int32, device="cuda")
    out = torch.ops.dtb200.joint_attention(q.cuda(), k.cuda(), v.cuda(), kv_len, None)
    dtb200.check_device_status("cuda")
    err = (out.float().cpu() - O.attention_fp32(q, k, v, kv_len=kv_len)).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3
    torch.library.opcheck(torch.ops.dtb200.joint_attention.default, (q.cuda(), k.cuda(), v.cuda(), kv_len, None),
                          test_utils=("test_schema", "test_faketensor"))


def test_dispatch_hook_layout_and_fallback_rules():
    q, k, v = _rand(1, 2, 1280, 2)
    bshd = [t.transpose(1, 2).contiguous().cuda() for t in (q, k, v)]      # (B, seq, heads, dim) as diffusers passes
    out = torch_op.dispatch(*bshd)
    dtb200.check_device_status("cuda")
    assert out.shape == bshd[0].shape
    err = (out.transpose(1, 2).float().cpu() - O.attention_fp32(q, k, v)).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3
    with pytest.raises(NotImplementedError):          # causal calls go to the stock path, which is absent here
        torch_op.dispatch(*bshd, is_causal=True)


@pytest.mark.parametrize("mode", ["ulysses", "ring"])
def test_two_gpu_drivers(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(ROOT, "tests", "multi_gpu_check.py"), mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PARITY OK" in r.stdout
