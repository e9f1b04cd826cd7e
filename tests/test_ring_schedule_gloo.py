"""The ring schedule on CPU ranks (gloo, world 2 and 4): every rank follows ring_step_plan() -- the very
function run_ring_fwd() follows on the GPU -- exchanging real shards with torch.distributed send/recv into
two alternating receive buffers, computing each step with the oracle and merging.  Checks that sends and
receives pair up (no rank blocks), that the double buffer is never overwritten before it is read, that the
causal skip ships only what is read, and that the merged result equals plain attention."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, causal, skip, out_dir):
    sys.path.insert(0, ROOT)
    import ctypes
    import torch
    import torch.distributed as dist
    from oracle import oracle
    from ringattention_b200 import _lib, synthetic
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = _lib.load()
    B, H, D, Sl = 1, 2, 64, 128
    S = Sl * world
    scale = D ** -0.5
    q, k, v = synthetic.make_qkv(77, B, H, D, rank * Sl, Sl)
    own = torch.from_numpy(np.stack([k, v]).view(np.int16).copy())
    recv = [torch.full_like(own, 0x7e00), torch.full_like(own, 0x7e00)]  # NaN-poisoned fp16 bit patterns
    acc = None
    sent_bytes = 0
    for s in range(world):
        plan = _lib.RingStepPlan()
        assert lib.ring_step_plan(world, rank, s, int(causal), int(skip), ctypes.byref(plan)) == 0
        ops = []
        if plan.do_send:
            ops.append(dist.P2POp(dist.isend, own, plan.send_to))
            sent_bytes += own.numel() * 2
        if plan.do_recv:
            ops.append(dist.P2POp(dist.irecv, recv[plan.recv_buffer], plan.recv_from))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        if plan.compute:
            buf = own if plan.compute_buffer < 0 else recv[plan.compute_buffer]
            kk, vv = (np.ascontiguousarray(buf[i].numpy().view(np.float16)) for i in (0, 1))
            assert not np.isnan(kk).any(), "step read a receive buffer that was never filled"
            part = oracle.attention_fwd(q, kk, vv, scale, causal, rank * Sl, plan.src_rank * Sl)
            acc = part if acc is None else oracle.lse_merge(acc[0], acc[1], part[0], part[1])
        for r in reqs:
            r.wait()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), o=acc[0], lse=acc[1], sent=np.int64(sent_bytes))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,causal,skip", [(2, False, 1), (4, False, 1), (4, True, 1), (4, True, 0), (2, True, 1)])
def test_ring_schedule_on_gloo_ranks(tmp_path, world, causal, skip):
    import torch.multiprocessing as mp
    from oracle import oracle
    from ringattention_b200 import synthetic
    port = _free_port()
    mp.spawn(_worker, args=(world, port, causal, skip, str(tmp_path)), nprocs=world, join=True)
    B, H, D, Sl = 1, 2, 64, 128
    q, k, v = synthetic.make_qkv(77, B, H, D, 0, Sl * world)
    want_o, want_lse = oracle.attention_fwd(q, k, v, D ** -0.5, causal)
    total_sent = 0
    for r in range(world):
        got = np.load(os.path.join(str(tmp_path), f"rank{r}.npz"))
        assert np.abs(got["o"] - want_o[:, :, r * Sl:(r + 1) * Sl]).max() <= 2e-6
        assert np.abs(got["lse"] - want_lse[:, :, r * Sl:(r + 1) * Sl]).max() <= 2e-6
        total_sent += int(got["sent"])
    shard = 2 * B * H * Sl * D * 2
    expect = world * (world - 1) * shard
    if causal and skip:
        expect //= 2  # only shards at or before the reader's own are shipped
    assert total_sent == expect


def test_step_plan_properties():
    import ctypes
    from ringattention_b200 import _lib
    lib = _lib.load()
    for world in (1, 2, 3, 4, 8):
        for causal in (0, 1):
            for skip in (0, 1):
                plans = [[_lib.RingStepPlan() for _ in range(world)] for _ in range(world)]
                for r in range(world):
                    for s in range(world):
                        assert lib.ring_step_plan(world, r, s, causal, skip, ctypes.byref(plans[r][s])) == 0
                for r in range(world):
                    assert sorted(p.src_rank for p in plans[r]) == list(range(world))  # every shard visited once
                    assert plans[r][0].src_rank == r and plans[r][0].compute_buffer == -1
                    for s in range(world):
                        p = plans[r][s]
                        assert p.compute == (0 if (causal and p.src_rank > r) else 1)
                        if s < world - 1:
                            peer = plans[p.send_to][s]           # the receiver expects exactly this sender
                            assert peer.recv_from == r and peer.do_recv == p.do_send
                            nxt = plans[r][s + 1]
                            assert nxt.src_rank == p.recv_from and nxt.compute_buffer == p.recv_buffer
                            assert nxt.compute <= p.do_recv        # whatever is computed was received
                        else:
                            assert p.do_send == 0 and p.do_recv == 0
    bad = _lib.RingStepPlan()
    assert lib.ring_step_plan(2, 2, 0, 0, 1, ctypes.byref(bad)) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_step_plan(2, 0, 2, 0, 1, ctypes.byref(bad)) == _lib.RING_ERR_INVALID_ARGUMENT
