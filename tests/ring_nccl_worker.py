"""One rank of a multi-GPU ring-attention parity run (launched by torchrun, one process per GPU).

Every rank builds its shard of the seeded global tensors, runs the ring forward three times (the later runs
reuse the receive buffers), then checks seeded sample rows of ITS OWN output shard against the fp64 oracle
evaluated over the full global K/V of the sampled heads.  Errors are max-reduced; rank 0 writes a JSON result.
The input generation and the check are the ones bench.py uses for its `parity` and `configs` objects.

Configurations are BASELINE.json's multi-GPU cases at full size (c2..c5) plus small ones, among them shards of
different lengths per rank (the reference's seqlen[], csrc/ring.h:9, csrc/ring_attention.cu:463,531) and bf16
inputs (csrc/kernel_traits.h:27-30).
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

UNEVEN = [640, 200, 1024, 333, 128, 77, 512, 900]   # rows per rank (first `world` entries)


def small_configs(world: int) -> dict:
    return {
        "small": dict(B=1, H=4, S=512 * world, D=128, causal=False, gain=1.0, heads=2, rows=48),
        "small_causal": dict(B=2, H=2, S=256 * world, D=64, causal=True, gain=1.0, heads=2, rows=48),
        "small_zigzag": dict(B=1, H=4, S=512 * world, D=128, causal=True, gain=1.0, heads=2, rows=48, zigzag=True),
        "uneven": dict(B=1, H=3, S=sum(UNEVEN[:world]), D=128, causal=False, gain=1.0, heads=2, rows=48, seqlens=UNEVEN[:world]),
        "uneven_causal": dict(B=2, H=2, S=sum(UNEVEN[:world]), D=64, causal=True, gain=1.0, heads=2, rows=48, seqlens=UNEVEN[:world]),
        "bf16": dict(B=1, H=4, S=512 * world, D=128, causal=False, gain=1.0, heads=2, rows=48, bf16=True),
        "bf16_causal_d64": dict(B=1, H=4, S=384 * world, D=64, causal=True, gain=1.0, heads=2, rows=48, bf16=True),
    }


def main():
    import bench
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--merge-mode", type=int, default=1)
    ap.add_argument("--out", default="")
    ap.add_argument("--transport", default="default", choices=["default", "nccl", "peer"])
    ap.add_argument("--recv-buffers", type=int, default=2)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import ringattention_b200 as ra

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rig = bench.Rig(torch, dist, dev, rank, world)
    table = dict(small_configs(world))
    table.update({n: c for n, c in bench.CONFIGS.items() if c["world"] == world})
    if args.config not in table:
        raise SystemExit(f"config {args.config} is not defined for world {world}")
    cfg = table[args.config]
    seed = 4321
    q, k, v, segs, seqlens = bench.make_rank_inputs(rig, cfg, seed)
    Sl = seqlens[rank]
    out = torch.full((cfg["B"], cfg["H"], Sl, cfg["D"]), float("nan"), device=dev)
    lse = torch.full((cfg["B"], cfg["H"], Sl), float("nan"), device=dev)
    ctx = ra.RingContext.from_torch_distributed()
    if args.transport != "default":
        ctx.set_option(ra.RING_OPT_TRANSPORT, ra.RING_TRANSPORT_NCCL if args.transport == "nccl" else ra.RING_TRANSPORT_PEER_COPY)
    transport = "peer" if ctx.get_option(ra.RING_OPT_TRANSPORT) == ra.RING_TRANSPORT_PEER_COPY else "nccl"
    ctx.set_option(ra.RING_OPT_MERGE_MODE, args.merge_mode)
    ctx.set_option(ra.RING_OPT_RECV_BUFFERS, args.recv_buffers)
    ctx.set_option(ra.RING_OPT_RECORD_TIMINGS, 1)
    ctx.set_option(ra.RING_OPT_CAUSAL_ZIGZAG, int(bool(cfg.get("zigzag"))))
    for _ in range(3):
        out.fill_(float("nan")); lse.fill_(float("nan"))
        ctx.forward(q, k, v, out, lse, causal=cfg["causal"], softmax_scale=cfg["D"] ** -0.5, seqlens=seqlens)
        ctx.synchronize()
    compute_ms, comm_ms, exposed_ms = ctx.timings()
    par = bench.check_parity(rig, cfg, seed, q, out, lse, segs, cfg["heads"], cfg["rows"])
    tmax = rig.reduce([sum(compute_ms), sum(exposed_ms)], "max")
    if rank == 0:
        res = {"config": args.config, "world": world, "B": cfg["B"], "H": cfg["H"], "S": cfg["S"], "D": cfg["D"],
               "causal": cfg["causal"], "seqlens": seqlens, "merge_mode": args.merge_mode, "transport": transport,
               "max_abs_o": par["max_abs_o"], "rel_l2_o": par["rel_l2_o"], "max_abs_lse": par["max_abs_lse"], "ok": par["ok"],
               "rank0_compute_ms": compute_ms, "rank0_comm_ms": comm_ms, "rank0_exposed_ms": exposed_ms,
               "max_rank_compute_ms": tmax[0], "max_rank_exposed_ms": tmax[1], "launches": ra.kernel_launch_count()}
        print(json.dumps(res), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f)
    ctx.destroy()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if par["ok"] else 1)


if __name__ == "__main__":
    main()
