"""Block-sparse attention: parity with the masked CPU oracle and the invariants the reference states."""
import pytest
import torch

import dtb200
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(B, H, S, seed, gain=2.0):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, H, S, 128, generator=g) for _ in range(3))
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True)) * gain).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    return q, k, v.to(torch.bfloat16)


def _check(out, ref):
    dtb200.check_device_status(DEV)
    err = (out.float().cpu() - ref).abs()
    assert not torch.isnan(out.float()).any()
    assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())


def test_full_table_is_bit_exact_with_dense():
    # "A full table is bit-exact with the dense kernel" (sparse_splash.py:1-5), online and bounded-logit paths
    S = 1100
    q, k, v = _rand(2, 3, S, 1)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    n_q, n_kv = (S + 511) // 512, (S + 255) // 256
    full = [list(range(n_kv)) for _ in range(n_q)]
    tb = dtb200.make_block_table(full, seq_q=S, seq_kv=S, block_q=512, block_kv=256)
    for kw in ({}, {"use_fixed_m": True}):
        dense = dtb200.attention(qd, kd, vd, kv_len=[S, 900], num_splits=1, **kw)   # same tile order, no split-KV
        sparse = dtb200.sparse_attention(qd, kd, vd, kv_table=tb, kv_len=[S, 900], **kw)
        dtb200.check_device_status(DEV)
        assert torch.equal(dense, sparse)


def test_windowed_table_matches_masked_oracle():
    S, bq, bkv = 1536, 256, 128
    q, k, v = _rand(1, 2, S, 2)
    n_q, n_kv = S // bq, S // bkv
    # a temporal-window style layout: each query block sees the first key block and a band around itself
    table = [sorted({0} | {kb for kb in range(n_kv) if abs(kb * bkv - qb * bq) <= 384}) for qb in range(n_q)]
    tb = dtb200.make_block_table(table, seq_q=S, seq_kv=S, block_q=bq, block_kv=bkv)
    out = dtb200.sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_table=tb)
    _check(out, O.attention_fp32(q, k, v, mask=O.block_mask(table, S, S, bq, bkv)))


def test_coarse_reference_blocks_head_classes_padding_and_empty_rows():
    S, bq, bkv = 2000, 512, 256          # reference-sized blocks, ragged sequence
    q, k, v = _rand(2, 4, S, 3)
    n_q, n_kv = (S + bq - 1) // bq, (S + bkv - 1) // bkv
    g = torch.Generator().manual_seed(7)
    classes = []
    for c in range(2):
        t = [sorted(torch.randperm(n_kv, generator=g)[: int(torch.randint(1, n_kv + 1, (1,), generator=g))].tolist())
             for _ in range(n_q)]
        classes.append(t)
    classes[1][2] = []                    # a query block that attends to nothing
    head_class = [0, 1, 1, 0]
    tb = dtb200.make_block_table((classes, head_class), seq_q=S, seq_kv=S, block_q=bq, block_kv=bkv, heads=4)
    kv_len = [S, 1300]
    out = dtb200.sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_table=tb, kv_len=kv_len)
    masks = [O.block_mask(classes[c], S, S, bq, bkv) for c in head_class]
    _check(out, O.attention_fp32(q, k, v, kv_len=kv_len, mask=masks))
    assert out[:, 1, 2 * bq:3 * bq].abs().max().item() == 0.0       # the empty row gives zeros
    assert out[1, :, 1300:].abs().max().item() == 0.0                # padded queries still come back as zeros


def test_table_shape_is_validated():
    q, k, v = _rand(1, 1, 512, 4)
    tb = dtb200.make_block_table([[0], [1]], seq_q=512, seq_kv=512, block_q=256, block_kv=256)
    with pytest.raises(ValueError):
        dtb200.sparse_attention(q[:, :, :256].contiguous().to(DEV), k.to(DEV), v.to(DEV), kv_table=tb)
    with pytest.raises(NotImplementedError):
        dtb200.make_block_table([[0]], seq_q=100, seq_kv=100, block_q=100, block_kv=100)
