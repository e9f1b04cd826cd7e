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
