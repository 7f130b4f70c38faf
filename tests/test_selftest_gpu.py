"""Hardware self-tests of the tensor-memory, TMA-swizzle and MMA-descriptor encodings (B200 only)."""
import pytest
import torch

from dtb200 import _lib

pytestmark = pytest.mark.gpu


def _run(fn, *tensors):
    dev = torch.device("cuda")
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    st = fn(*[t.data_ptr() for t in tensors], status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(st, fn.__name__)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]


def test_tmem_roundtrip_is_bit_exact():
    x = torch.randn(128, 128, device="cuda")
    y = torch.zeros_like(x)
    _run(_lib.load().dtb_selftest_tmem_roundtrip, x, y)
    assert torch.equal(x, y)


def test_qk_tile_matches_matmul():
    q = torch.randn(128, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(128, 128, device="cuda").to(torch.bfloat16)
    s = torch.zeros(128, 128, device="cuda")
    _run(_lib.load().dtb_selftest_qk, q, k, s)
    torch.testing.assert_close(s, q.float() @ k.float().T, rtol=1e-5, atol=1e-4)


def test_pv_tile_matches_matmul_with_asymmetric_data():
    p = torch.rand(128, 128, device="cuda").to(torch.bfloat16)
    v = (torch.randn(128, 128, device="cuda") + torch.arange(128, device="cuda")[None, :] * 0.01).to(torch.bfloat16)
    o = torch.zeros(128, 128, device="cuda")
    _run(_lib.load().dtb_selftest_pv, p, v, o)
    torch.testing.assert_close(o, p.float() @ v.float(), rtol=1e-5, atol=1e-4)


def test_bounded_wait_gives_up_and_reports():
    """A wait nothing will satisfy must end by itself, report where it gave up and leave the GPU usable."""
    import time

    lib = _lib.load()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    _lib.check(lib.dtb_selftest_wait_timeout(50_000_000, 77, status.data_ptr(), returned.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream), "dtb_selftest_wait_timeout")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert returned.item() == 2
    st = status.tolist()
    assert st[0] == 1 and st[1] == 77 and st[2] == 0
    # the context is intact: ordinary work still runs
    x = torch.randn(128, 128, device="cuda")
    y = torch.zeros_like(x)
    _run(lib.dtb_selftest_tmem_roundtrip, x, y)
    assert torch.equal(x, y)
