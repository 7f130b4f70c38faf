"""The allocation-free entry point, `dtb_attn_fwd_static_scratch`, called through the C ABI.

Some hosts of this library can hand it input and output buffers but no scratch: a handler running
inside another runtime's execution callback (an XLA FFI custom call, a serving engine's plugin slot) or
a foreign-language binding that never sees a device allocator.  For them the split-KV partials live in
an array built into the library.  This file checks that the entry point gives the same output as the
ordinary `dtb_attn_fwd` with a caller-provided workspace, twice in a row on different shapes (the array
keeps the previous call's contents), that it refuses calls whose partials would not fit, and that it
leaves the amount of free device memory unchanged.

It sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

import dtb200
from dtb200 import _lib, ops
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(B, H, Sq, Skv, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Sq, 128, generator=g)
    k = torch.randn(B, H, Skv, 128, generator=g)
    v = torch.randn(B, H, Skv, 128, generator=g)
    q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True)) * 3.0).to(torch.bfloat16)
    k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True))).to(torch.bfloat16)
    return q.to(DEV), k.to(DEV), v.to(torch.bfloat16).to(DEV)


def _static_scratch_call(q, k, v, kv_len, num_splits):
    dev = q.device
    out = torch.empty_like(q)
    kv_len_t = ops._kv_len_tensor(kv_len, q.shape[0], dev)
    flags = _lib.FLAG_ZERO_PADDED_ROWS if kv_len_t is not None else 0
    p = ops._fill_params(q, k, v, out, kv_len_t, None, None, flags, num_splits, ops._status_buffer(dev))
    st = _lib.load().dtb_attn_fwd_static_scratch(ctypes.byref(p), torch.cuda.current_stream(dev).cuda_stream)
    return st, out


def test_static_scratch_matches_workspace_path_twice_in_a_row():
    cases = [
        # (B, H, Sq, Skv, kv_len, splits): the second call is smaller, so stale partials of the first
        # remain in the array beyond what it writes
        (2, 4, 300, 4096, [4000, 2500], 6),
        (1, 2, 128, 2048, None, 3),
    ]
    free_after_first = None
    for i, (B, H, Sq, Skv, kv_len, splits) in enumerate(cases):
        q, k, v = _inputs(B, H, Sq, Skv, seed=40 + i)
        want = dtb200.attention(q, k, v, kv_len=kv_len, num_splits=splits)      # caller-provided workspace
        dtb200.check_device_status(DEV)
        st, got = _static_scratch_call(q, k, v, kv_len, splits)
        _lib.check(st, "dtb_attn_fwd_static_scratch")
        dtb200.check_device_status(DEV)
        # same kernels, same split boundaries, same merge order: the outputs are bit-identical,
        # which is well inside the path's tolerance (max-abs 2e-2, mean-abs 2e-3)
        err = (got.float() - want.float()).abs()
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3
        assert torch.equal(got, want)
        # and both are right: the fp32 oracle on the same inputs
        err = (got.float().cpu() - O.attention_fp32(q, k, v, kv_len=kv_len)).abs()
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3
        free_now = torch.cuda.mem_get_info()[0]
        if free_after_first is None:
            free_after_first = free_now
        else:
            st, _ = _static_scratch_call(q, k, v, kv_len, splits)
            _lib.check(st, "dtb_attn_fwd_static_scratch")
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] >= free_now - (1 << 20)     # the call itself allocated nothing


def test_static_scratch_rejects_oversized_calls_without_launching():
    # 8 splits x 2 x 24 x 512 rows x 130 floats = 102 MB of partials: more than the built-in 32 MiB
    q, k, v = _inputs(2, 24, 512, 8192, seed=50)
    st, out = _static_scratch_call(q, k, v, None, 8)
    assert st == 6                                           # DTB_ERR_WORKSPACE
    detail = _lib.load().dtb_last_error_detail().decode()
    assert str(_lib.STATIC_SCRATCH_BYTES) in detail
    with pytest.raises(ValueError):
        _lib.check(st, "dtb_attn_fwd_static_scratch")


def test_static_scratch_unsplit_call_needs_no_scratch():
    q, k, v = _inputs(1, 8, 1024, 1024, seed=51)
    st, got = _static_scratch_call(q, k, v, 1000, 1)
    _lib.check(st, "dtb_attn_fwd_static_scratch")
    want = dtb200.attention(q, k, v, kv_len=1000, num_splits=1)
    dtb200.check_device_status(DEV)
    assert torch.equal(got, want)


def test_static_scratch_with_automatic_split_selection():
    """num_splits = 0: the library picks the split itself (a short-query call that leaves most SMs idle
    unsplit) and sizes its use of the built-in array accordingly.  Twice in a row, against the ordinary entry
    point and the fp32 oracle."""
    q, k, v = _inputs(1, 2, 256, 8192, seed=52)
    p = ops._fill_params(q, k, v, torch.empty_like(q), None, None, None, 0, 0, None)
    assert _lib.load().dtb_attn_workspace_bytes(ctypes.byref(p)) > 0          # the automatic choice does split this call
    want = dtb200.attention(q, k, v, kv_len=[8000], num_splits=0)
    ref = O.attention_fp32(q, k, v, kv_len=[8000])
    for _ in range(2):
        st, got = _static_scratch_call(q, k, v, [8000], 0)
        _lib.check(st, "dtb_attn_fwd_static_scratch")
        dtb200.check_device_status(DEV)
        for other in (want.float().cpu(), ref):
            err = (got.float().cpu() - other).abs()
            assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3
