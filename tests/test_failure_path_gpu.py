"""The bounded-wait error path on a real GPU, without faulting it.

Every device-side wait of the library gives up after a number of SM clocks, records its site
and lets the kernel return.  The library's self-test kernel makes one such wait run out (a
barrier that nothing arrives on, limit ~0.5 ms); the test checks that the kernel returns, that
rt_check_device() turns the error word into RT_ERR_DEVICE_WAIT with the site id, that the word
is cleared afterwards, and that the next real kernel launch works."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi, ops
    ops.check_device()                                   # clean start
    t0 = time.perf_counter()
    ops.selftest_bounded_wait(limit_cycles=1_000_000, target=0)
    torch.cuda.synchronize()                             # the kernel returned by itself
    assert time.perf_counter() - t0 < 5.0
    with pytest.raises(capi.RtError) as e:
        ops.check_device()
    assert e.value.code == 4 and "site 901" in str(e.value)
    ops.check_device()                                   # reported once, then cleared
    # the context is intact: a tensor-core GEMM right after gives the right answer
    a = torch.randn(256, 128, device="cuda").to(torch.bfloat16)
    w = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
    out = ops.gemm(a, w)
    assert (out.float() - a.float() @ w.float().t()).abs().max().item() < 0.25
    ops.check_device()


def test_selftest_rejects_unbounded_limits():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi, ops
    for bad in (0, -5, 10**12):
        with pytest.raises(capi.RtError):
            ops.selftest_bounded_wait(limit_cycles=bad)
