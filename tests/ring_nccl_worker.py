"""One rank of a multi-GPU ring-attention parity run (launched by torchrun, one process per GPU).

Every rank builds its shard of the seeded global tensors, runs the NCCL ring forward twice (the second run
reuses the receive buffers), then checks seeded sample rows of ITS OWN output shard against the fp64 oracle
evaluated over the full global K/V of the sampled heads.  Errors are max-reduced; rank 0 writes a JSON result.

Configurations are BASELINE.json's multi-GPU cases at full size (c2..c5) plus small ones.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

CONFIGS = {
    # name: (world, B, H, S_total, D, causal, gain, sampled heads, sample rows per head)
    "small": (None, 1, 4, None, 128, False, 1.0, 2, 48),       # S_total = 512 * world
    "small_causal": (None, 2, 2, None, 64, True, 1.0, 2, 48),  # S_total = 256 * world
    "c2": (2, 2, 16, 8192, 128, False, 1.0, 3, 64),
    "c3": (4, 1, 32, 32768, 128, False, 0.5, 3, 64),
    "c4": (8, 1, 32, 131072, 128, True, 1.0, 2, 48),
    "c4_zigzag": (8, 1, 32, 131072, 128, True, 1.0, 2, 48),     # same problem, zig-zag sharding
    "small_zigzag": (None, 1, 4, None, 128, True, 1.0, 2, 48),  # S_total = 512 * world
    "c5": (8, 1, 8, 1048576, 128, False, 1.0, 1, 24),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=sorted(CONFIGS))
    ap.add_argument("--merge-mode", type=int, default=1)
    ap.add_argument("--out", default="")
    ap.add_argument("--transport", default="default", choices=["default", "nccl", "peer"])
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import ringattention_b200 as ra
    from ringattention_b200 import synthetic
    from oracle import oracle
    from tests.gpu_util import TOL_LSE, TOL_O_MAXABS, TOL_O_RELL2

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cw, B, H, S, D, causal, gain, n_heads, n_rows = CONFIGS[args.config]
    if cw is not None and cw != world:
        raise SystemExit(f"config {args.config} needs world {cw}, got {world}")
    if S is None:
        S = (256 if args.config == "small_causal" else 512) * world
    zigzag = args.config.endswith("zigzag")
    Sl = S // world
    seed = 4321
    scale = D ** -0.5

    t0 = time.time()
    if zigzag:  # this rank's rows: chunk `rank` then chunk `2 * world - 1 - rank`
        my_rows = synthetic.zigzag_rows(rank, world, S)
        ch = Sl // 2
        parts = [synthetic.make_qkv(seed, B, H, D, int(my_rows[0]), ch, gain), synthetic.make_qkv(seed, B, H, D, int(my_rows[ch]), ch, gain)]
        q, k, v = (torch.from_numpy(np.concatenate([parts[0][i], parts[1][i]], axis=2)).to(dev) for i in range(3))
    else:
        my_rows = np.arange(rank * Sl, (rank + 1) * Sl)
        q, k, v = (torch.from_numpy(x).to(dev) for x in synthetic.make_qkv(seed, B, H, D, rank * Sl, Sl, gain))
    t_gen = time.time() - t0
    out = torch.full((B, H, Sl, D), float("nan"), device=dev)
    lse = torch.full((B, H, Sl), float("nan"), device=dev)
    ctx = ra.RingContext.from_torch_distributed()
    if args.transport != "default":
        ctx.set_option(ra.RING_OPT_TRANSPORT, ra.RING_TRANSPORT_NCCL if args.transport == "nccl" else ra.RING_TRANSPORT_PEER_COPY)
    transport = "peer" if ctx.get_option(ra.RING_OPT_TRANSPORT) == ra.RING_TRANSPORT_PEER_COPY else "nccl"
    ctx.set_option(ra.RING_OPT_MERGE_MODE, args.merge_mode)
    ctx.set_option(ra.RING_OPT_RECORD_TIMINGS, 1)
    ctx.set_option(ra.RING_OPT_CAUSAL_ZIGZAG, int(zigzag))
    for _ in range(3):
        out.fill_(float("nan")); lse.fill_(float("nan"))
        ctx.forward(q, k, v, out, lse, causal=causal, softmax_scale=scale)
        ctx.synchronize()
    compute_ms, comm_ms, exposed_ms = ctx.timings()

    # ---- sampled rows of this rank's shard against the fp64 oracle over the full K/V of their head ----
    rng = np.random.Generator(np.random.Philox(key=np.array([seed, rank], dtype=np.uint64)))
    heads = sorted({(int(rng.integers(0, B)), int(rng.integers(0, H))) for _ in range(n_heads)})
    err_o = err_l = 0.0
    num = den = 0.0
    t0 = time.time()
    o_host, l_host = out.cpu().numpy(), lse.cpu().numpy()
    assert not np.isnan(o_host).any() and not np.isnan(l_host).any(), "unwritten output rows"
    for (b, h) in heads:
        idx = np.unique(np.concatenate([[0, Sl - 1, Sl // 2], rng.integers(0, Sl, n_rows)])).astype(np.int64)
        kf = synthetic.make_head("k", seed, H, D, b, h, 0, S, gain)[None, None]
        vf = synthetic.make_head("v", seed, H, D, b, h, 0, S, gain)[None, None]
        qh = np.ascontiguousarray(q[b, h].cpu().numpy())[None, None]
        rows = np.stack([np.zeros_like(idx), np.zeros_like(idx), idx], axis=1)
        # global index of local row i: my_rows[i] (one run of rows, or two under zig-zag sharding)
        want_o = np.empty((len(idx), D), np.float32); want_l = np.empty(len(idx), np.float32)
        cut = Sl // 2
        for part in (0, 1):
            sel = (idx >= cut) if part else (idx < cut)
            if sel.any():
                off = int(my_rows[part * cut]) - part * cut
                want_o[sel], want_l[sel] = oracle.attention_rows(qh, kf, vf, rows[sel], scale, causal, q_off=off, k_off=0)
        got_o, got_l = o_host[b, h, idx], l_host[b, h, idx]
        err_o = max(err_o, float(np.abs(got_o - want_o).max()))
        err_l = max(err_l, float(np.abs(got_l - want_l).max()))
        num += float(((got_o - want_o) ** 2).sum()); den += float((want_o ** 2).sum())
    t_oracle = time.time() - t0
    stats = torch.tensor([err_o, err_l, num, den], dtype=torch.float64, device=dev)
    mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    tm = torch.tensor([sum(compute_ms), sum(exposed_ms)], dtype=torch.float64, device=dev)
    tmax = tm.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    rel = float((sm[2] / sm[3]).sqrt())
    ok = bool(mx[0] <= TOL_O_MAXABS and rel <= TOL_O_RELL2 and mx[1] <= TOL_LSE)
    if rank == 0:
        res = {"config": args.config, "world": world, "B": B, "H": H, "S": S, "D": D, "causal": causal,
               "merge_mode": args.merge_mode, "transport": transport, "max_abs_o": float(mx[0]), "rel_l2_o": rel, "max_abs_lse": float(mx[1]),
               "ok": ok, "rank0_compute_ms": compute_ms, "rank0_comm_ms": comm_ms, "rank0_exposed_ms": exposed_ms,
               "max_rank_compute_ms": float(tmax[0]), "max_rank_exposed_ms": float(tmax[1]),
               "gen_s": t_gen, "oracle_s": t_oracle, "launches": ra.kernel_launch_count()}
        print(json.dumps(res), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f)
    ctx.destroy()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
