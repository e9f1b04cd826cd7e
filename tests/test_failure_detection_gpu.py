"""Failure detection without faulting the GPU: a bounded wait that runs out, and a status word set from the host."""
import ctypes

import numpy as np
import pytest

from ringattention_b200 import _lib, synthetic
from tests.gpu_util import to_dev

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports():
    """The kernels' mbarrier wait, on a barrier nothing completes: returns after ~2 s with the code recorded."""
    lib = _lib.load()
    status, ms = ctypes.c_int(0), ctypes.c_float(0)
    assert lib.ring_selftest_wait_timeout(121, ctypes.byref(status), ctypes.byref(ms)) == 0, lib.ring_last_error_string()
    assert status.value == 121
    assert 1500.0 <= ms.value <= 6000.0
    # the context is still usable: nothing faulted
    st = ctypes.c_int(-1)
    assert lib.ring_device_status(ctypes.byref(st)) == 0 and st.value == 0


def test_recorded_failure_stops_later_kernels_until_reset():
    import torch
    import ringattention_b200 as ra
    B, H, S, D = 1, 2, 256, 64
    q, k, v = (to_dev(x) for x in synthetic.make_qkv(9, B, H, D, 0, S))
    out = torch.full((B, H, S, D), float("nan"), device="cuda")
    lse = torch.full((B, H, S), float("nan"), device="cuda")
    ctx = ra.RingContext.create(0, 1, None)
    ra.device_status_reset()
    assert _lib.load().ring_device_status_inject(113) == 0
    ctx.forward(q, k, v, out, lse)
    with pytest.raises(ra.RingError) as e:
        ctx.synchronize()
    assert e.value.code == _lib.RING_ERR_DEVICE_TIMEOUT and "113" in str(e.value)
    assert torch.isnan(out).all()          # every CTA returned before touching its output
    ra.device_status_reset()
    ctx.forward(q, k, v, out, lse)
    ctx.synchronize()
    assert not torch.isnan(out).any() and ra.device_status() == 0
    ctx.destroy()


def test_host_deadline_notices_a_forward_that_does_not_finish():
    """A forward queued behind a stream wait that nothing satisfies yet (what a stopped peer looks like from this
    rank's side: a stream waiting for a flag): synchronize(timeout_ms) gives up on time and says so, nothing on the
    device is disturbed, and once the flag is written the same forward completes with correct results."""
    import time

    import torch
    import ringattention_b200 as ra
    from cuda.bindings import driver
    from oracle import oracle

    B, H, S, D = 1, 2, 256, 64
    qh, kh, vh = synthetic.make_qkv(21, B, H, D, 0, S)
    q, k, v = (to_dev(x) for x in (qh, kh, vh))
    out = torch.zeros((B, H, S, D), device="cuda")
    lse = torch.zeros((B, H, S), device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ra.device_status_reset()
    ctx = ra.RingContext.create(0, 1, None)
    work, side = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    released = False
    try:
        (err,) = driver.cuStreamWaitValue32(work.cuda_stream, flag.data_ptr(), 1, driver.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ)
        assert int(err) == 0
        ctx.forward(q, k, v, out, lse, stream=work.cuda_stream)
        t0 = time.perf_counter()
        with pytest.raises(ra.RingError) as e:
            ctx.synchronize(timeout_ms=300)
        waited = time.perf_counter() - t0
        assert e.value.code == ra.RING_ERR_HOST_TIMEOUT and "compute" in str(e.value)
        assert 0.25 <= waited <= 2.0
        with torch.cuda.stream(side):
            flag.fill_(1)
        released = True
        ctx.synchronize(timeout_ms=10000)   # now it finishes
    finally:
        if not released:
            with torch.cuda.stream(side):
                flag.fill_(1)
        torch.cuda.synchronize()
    want_o, want_lse = oracle.attention_fwd(qh, kh, vh, D ** -0.5)
    assert np.abs(out.cpu().numpy() - want_o).max() <= 2e-3
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 1e-4
    ctx.destroy()


def test_abort_after_host_timeout_lets_the_context_go():
    """The way out after a detected failure: a forward sits behind a stream wait nothing satisfies (a stopped peer,
    seen from this rank); synchronize(timeout) reports it; abort() marks the context dead, further forwards are
    refused, and destroy() comes back within its own bounded drain instead of blocking on the device.  The flag is
    written afterwards, so nothing is left waiting on the GPU when the test ends."""
    import time

    import torch
    import ringattention_b200 as ra
    from cuda.bindings import driver

    B, H, S, D = 1, 2, 256, 64
    q, k, v = (to_dev(x) for x in synthetic.make_qkv(22, B, H, D, 0, S))
    out = torch.zeros((B, H, S, D), device="cuda")
    lse = torch.zeros((B, H, S), device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ra.device_status_reset()
    ctx = ra.RingContext.create(0, 1, None)
    work, side = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    try:
        (err,) = driver.cuStreamWaitValue32(work.cuda_stream, flag.data_ptr(), 1, driver.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ)
        assert int(err) == 0
        ctx.forward(q, k, v, out, lse, stream=work.cuda_stream)
        with pytest.raises(ra.RingError) as e:
            ctx.synchronize(timeout_ms=200)
        assert e.value.code == ra.RING_ERR_HOST_TIMEOUT
        ctx.abort()
        with pytest.raises(ra.RingError) as e:
            ctx.forward(q, k, v, out, lse, stream=work.cuda_stream)
        assert e.value.code == _lib.RING_ERR_UNSUPPORTED and "aborted" in str(e.value)
        t0 = time.perf_counter()
        ctx.destroy()                       # must not wait for the stream that is still held
        assert time.perf_counter() - t0 <= 8.0
    finally:
        with torch.cuda.stream(side):
            flag.fill_(1)
        torch.cuda.synchronize()
    assert ra.device_status() == 0
