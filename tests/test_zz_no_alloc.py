"""The entry point that allocates nothing (ring_attention_chunked_fwd_static), called through the C ABI.

Some hosts give a component its input and output tensors but no way to obtain device memory of its own
(a serving runtime that reserved the whole GPU, a fixed memory budget).  For them the library keeps the
scratch of the chunked forward in a fixed device array.  The checks: the result equals the existing
ring_attention_block_fwd over the whole K/V, and the CPU oracle, within the parity bar of this repository,
on calls in a row that share the array (second call: other shape, other data, so stale contents would
show); once the first call has done the one-time set-up, a further call leaves the device's free memory
exactly as it was while the kernel counter rises; the path's own status word reads zero; and sizes beyond
the array are refused.  Collected last on purpose (file name), so a failure here cannot hide
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

    from oracle import oracle

    def both(seed, B, H, Sq, Sk, D, chunk, causal):
        qh = synthetic.make_shard("q", seed, B, H, D, 0, Sq)
        kh = synthetic.make_shard("k", seed, B, H, D, 0, Sk)
        vh = synthetic.make_shard("v", seed, B, H, D, 0, Sk)
        q, k, v = (torch.from_numpy(x).cuda() for x in (qh, kh, vh))
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
        want_o, want_l = oracle.attention_fwd(qh, kh, vh, scale, causal=causal)   # fp64 accumulation on the CPU
        assert np.abs(want_o - b).max() <= TOL_O_MAXABS
        assert np.linalg.norm(want_o - b) / np.linalg.norm(want_o) <= TOL_O_RELL2
        assert np.abs(want_l - lb).max() <= TOL_LSE
        st = ctypes.c_int(-1)
        assert lib.ring_static_status(ctypes.byref(st), stream) == 0 and st.value == 0   # the word THIS path writes

    # two calls in a row through the same fixed array: different shapes, data, chunking and masks
    both(501, 1, 4, 512, 1024, 128, 256, False)
    both(502, 2, 2, 256, 640, 64, 256, True)      # last chunk shorter than the others
    both(501, 1, 4, 512, 1024, 128, 1024, False)  # single chunk: scratch untouched, still equal

    # Set-up is done (every head dimension used below has run once): one more call must not change the device's
    # free memory by a byte, although it launches kernels.  Inputs and outputs are made before the measurement.
    B, H, Sq, Sk, D = 1, 4, 512, 1024, 128
    q = torch.from_numpy(synthetic.make_shard("q", 503, B, H, D, 0, Sq)).cuda()
    k = torch.from_numpy(synthetic.make_shard("k", 503, B, H, D, 0, Sk)).cuda()
    v = torch.from_numpy(synthetic.make_shard("v", 503, B, H, D, 0, Sk)).cuda()
    o = torch.empty((B, H, Sq, D), device="cuda")
    l = torch.empty((B, H, Sq), device="cuda")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    launches0 = lib.ring_kernel_launch_count()
    rc = lib.ring_attention_chunked_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), l.data_ptr(),
                                               B, H, Sq, Sk, D, D ** -0.5, 0, 256, 0, stream)
    assert rc == 0, lib.ring_last_error_string()
    st = ctypes.c_int(-1)
    assert lib.ring_static_status(ctypes.byref(st), stream) == 0 and st.value == 0
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device free memory changed by {free0 - free1} bytes across a call"
    assert lib.ring_kernel_launch_count() - launches0 == 4 + 3   # four chunks, three merges
