"""Generates the committed golden vectors under tests/golden/.

The reference project has no fixtures for its attention kernel and cannot be run offline, so these
vectors pin the oracle against itself across time (a regression fixture): seeded inputs, the fp32
softmax output and the restated-reference output.  Regenerate with

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "diffusers-tpu_b200"))

from oracle import attn_oracle as O  # noqa: E402

CASES = {
    # name: (B, H, Hkv, Sq, Skv, kv_len per batch or None, q gain)
    "joint_small": (2, 1, 1, 160, 160, [160, 131], 1.0),
    "peaked_cross": (1, 2, 1, 130, 200, [177], 6.0),
}


def make_case(name):
    B, H, Hkv, Sq, Skv, kv_len, gain = CASES[name]
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    q = torch.randn(B, H, Sq, 128, generator=g)
    k = torch.randn(B, Hkv, Skv, 128, generator=g)
    v = torch.randn(B, Hkv, Skv, 128, generator=g)
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6) * gain).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    v = v.to(torch.bfloat16)
    return q, k, v, kv_len


def main():
    for name in CASES:
        q, k, v, kv_len = make_case(name)
        ref = O.attention_fp32(q, k, v, kv_len=kv_len)
        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"),
            q=q.view(torch.int16).numpy(), k=k.view(torch.int16).numpy(), v=v.view(torch.int16).numpy(),
            kv_len=np.asarray(kv_len, dtype=np.int32), out_fp32=ref.numpy().astype(np.float32),
        )
        print(name, "written", ref.shape)


if __name__ == "__main__":
    main()
