"""Two ranks, one GPU each: what a rank does when its peer stops taking part (launched by torchrun).

Nothing on a GPU is faulted, trapped or left spinning.  Rank 1 simply does not call the second forward; it keeps its
context (its receive buffers and flag block, which rank 0's copies still write to) alive behind a host barrier.  Rank
0's second forward then cannot finish: its exchange stream waits for a "buffer free" flag that rank 1 never writes.
Rank 0 notices on the host (synchronize with a deadline -> RING_ERR_HOST_TIMEOUT), calls abort(), which releases the
queued waits from the host and aborts the communicator, destroys its context within a bounded time and only then lets
rank 1 go.  Peer-copy transport; no NCCL kernel is ever waiting for a peer.  The rendezvous is gloo.
"""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import ringattention_b200 as ra
    from ringattention_b200 import synthetic

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    assert world == 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo")
    B, H, Sl, D = 1, 2, 512, 128
    q, k, v = (torch.from_numpy(x).to(dev) for x in synthetic.make_qkv(77, B, H, D, rank * Sl, Sl))
    out = torch.zeros((B, H, Sl, D), device=dev)
    lse = torch.zeros((B, H, Sl), device=dev)
    ctx = ra.RingContext.from_torch_distributed()
    if ctx.get_option(ra.RING_OPT_TRANSPORT) != ra.RING_TRANSPORT_PEER_COPY:
        print(json.dumps({"rank": rank, "skipped": "the peer-copy transport is not available between these GPUs"}), flush=True)
        ctx.destroy()
        dist.barrier()
        return
    ctx.forward(q, k, v, out, lse)          # a complete forward first: both ranks take part
    ctx.synchronize()
    dist.barrier()
    res = {"rank": rank}
    if rank == 0:
        ctx.forward(q, k, v, out, lse)      # rank 1 sits this one out
        t0 = time.perf_counter()
        try:
            ctx.synchronize(timeout_ms=500)
            res["timeout_code"] = 0
        except ra.RingError as e:
            res["timeout_code"] = e.code
            res["timeout_message"] = str(e)
        res["waited_s"] = time.perf_counter() - t0
        ctx.abort()
        try:
            ctx.forward(q, k, v, out, lse)
            res["refused_after_abort"] = False
        except ra.RingError as e:
            res["refused_after_abort"] = e.code == -6   # RING_ERR_UNSUPPORTED
        t0 = time.perf_counter()
        ctx.destroy()
        res["destroy_s"] = time.perf_counter() - t0
        torch.cuda.synchronize()            # the released work has drained: nothing is left waiting on this GPU
        res["device_status"] = ra.device_status()
    dist.barrier()                          # rank 1 kept its buffers mapped until here
    if rank == 1:
        ctx.abort()                         # its communicator lost its peer: abort rather than destroy it
        ctx.destroy()
        torch.cuda.synchronize()
        res["device_status"] = ra.device_status()
    print(json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
