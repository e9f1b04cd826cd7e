"""The entry point that allocates nothing (ring_attention_chunked_fwd_static), called through the C ABI.

Some hosts give a component its input and output tensors but no way to obtain device memory of its own
(a serving runtime that reserved the whole GPU, a fixed memory budget).  For them the library keeps the
scratch of the chunked forward in a fixed device array.  The checks: the result equals the existing
ring_attention_block_fwd over the whole K/V within the parity bar of this repository, on two calls in a
row that share the array (second call: other shape, other data, so stale contents would show), and sizes
beyond the array are refused.  Collected last on purpose (file name), so a failure here cannot hide
another test's result in a run that stops at the first failure.
"""
import ctypes

import numpy as np
import pytest

from ringattention_b200 import _lib, synthetic
from ringattention_b200 import build as lib_build

TOL_O_MAXABS, TOL_O_RELL2, TOL_LSE = 2e-3, 1e-3, 1e-4


def test_sizes_beyond_the_fixed_scratch_are_refused():
    lib_build.build()
    lib = _lib.load()
    # 65537 rows of 64 floats: one row too many (refused before any CUDA call)
    rc = lib.ring_attention_chunked_fwd_static(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 1, 1, 65536 + 128, 128, 64,
                                               0.125, 0, 128, 0, None)
    assert rc == _lib.RING_ERR_INVALID_ARGUMENT
    assert b"exceeds the fixed scratch" in lib.ring_last_error_string()
    # 4 Mi floats + one tile with dim 128
    rc = lib.ring_attention_chunked_fwd_static(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 1, 1, 32768 + 128, 128, 128,
                                               0.125, 0, 128, 0, None)
    assert rc == _lib.RING_ERR_INVALID_ARGUMENT
    rc = lib.ring_attention_chunked_fwd_static(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 1, 1, 128, 128, 128,
                                               0.125, 0, 100, 0, None)
    assert rc == _lib.RING_ERR_INVALID_ARGUMENT
    assert b"kv_chunk" in lib.ring_last_error_string()


@pytest.mark.gpu
def test_static_scratch_entry_matches_block_forward_twice():
    import torch
    lib_build.build()
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def both(seed, B, H, Sq, Sk, D, chunk, causal):
        q = torch.from_numpy(synthetic.make_shard("q", seed, B, H, D, 0, Sq)).cuda()
        k = torch.from_numpy(synthetic.make_shard("k", seed, B, H, D, 0, Sk)).cuda()
        v = torch.from_numpy(synthetic.make_shard("v", seed, B, H, D, 0, Sk)).cuda()
        scale = D ** -0.5
        o_ref = torch.full((B, H, Sq, D), float("nan"), device="cuda")
        l_ref = torch.full((B, H, Sq), float("nan"), device="cuda")
        rc = lib.ring_attention_block_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_ref.data_ptr(), l_ref.data_ptr(),
                                          B, H, Sq, Sk, D, scale, int(causal), 0, 0, 0, 0, stream)
        assert rc == 0, lib.ring_last_error_string()
        o_new = torch.full((B, H, Sq, D), float("nan"), device="cuda")
        l_new = torch.full((B, H, Sq), float("nan"), device="cuda")
        rc = lib.ring_attention_chunked_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_new.data_ptr(),
                                                   l_new.data_ptr(), B, H, Sq, Sk, D, scale, int(causal), chunk, 0, stream)
        assert rc == 0, lib.ring_last_error_string()
        torch.cuda.synchronize()
        a, b = o_ref.cpu().numpy(), o_new.cpu().numpy()
        la, lb = l_ref.cpu().numpy(), l_new.cpu().numpy()
        assert not np.isnan(b).any() and not np.isnan(lb).any()
        assert np.abs(a - b).max() <= TOL_O_MAXABS
        assert np.linalg.norm(a - b) / np.linalg.norm(a) <= TOL_O_RELL2
        assert np.abs(la - lb).max() <= TOL_LSE

    # two calls in a row through the same fixed array: different shapes, data, chunking and masks
    both(501, 1, 4, 512, 1024, 128, 256, False)
    both(502, 2, 2, 256, 640, 64, 256, True)      # last chunk shorter than the others
    both(501, 1, 4, 512, 1024, 128, 1024, False)  # single chunk: scratch untouched, still equal
    status = ctypes.c_int(-1)
    assert lib.ring_device_status(ctypes.byref(status)) == 0 and status.value == 0
