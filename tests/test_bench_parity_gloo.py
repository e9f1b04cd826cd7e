"""The multi-rank parity check that bench.py and the multi-GPU worker print (`parity` objects), run on CPU ranks
(gloo, world 2): every rank builds its shard with bench.make_rank_inputs -- contiguous, uneven and zig-zag shardings,
fp16 and bf16 -- fills its "output" with the oracle's full attention of its own rows, and bench.check_parity must
accept it; one wrong row on ONE rank, or rows left unwritten, must fail the check on EVERY rank (the result is
max-reduced), which is what makes a stale or misplaced K/V shard visible in the benchmark's line."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = {
    "even": dict(B=1, H=2, S=512, D=64, causal=False, gain=1.0),
    "uneven_causal": dict(B=2, H=2, S=320 + 192, D=64, causal=True, gain=1.0, seqlens=[320, 192]),
    "zigzag": dict(B=1, H=2, S=512, D=128, causal=True, gain=1.0, zigzag=True),
    "bf16": dict(B=1, H=2, S=384, D=64, causal=True, gain=1.0, bf16=True),
}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import bench
    from oracle import oracle
    from ringattention_b200 import synthetic
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    class CpuRig(bench.Rig):   # same reductions over gloo, tensors on the CPU
        def __init__(self):
            self.torch, self.dist, self.dev, self.rank, self.world = torch, dist, torch.device("cpu"), rank, world
            self.stream = None

        def barrier(self):
            dist.barrier()

    rig = CpuRig()
    res = {}
    for name, cfg in CASES.items():
        seed = 99
        q, k, v, segs, seqlens = bench.make_rank_inputs(rig, cfg, seed)
        S, D, gain = cfg["S"], cfg["D"], cfg["gain"]
        B, H = cfg["B"], cfg["H"]
        # the full global K/V, regenerated from the seed; this rank's rows attend to all of it
        kf, vf = (synthetic.make_shard(w, seed, B, H, D, 0, S, gain) for w in ("k", "v"))
        qn = q.view(torch.int16).numpy().view(np.uint16) if cfg.get("bf16") else q.numpy()
        if cfg.get("bf16"):
            kf, vf = (oracle.to_bf16_bits(x.astype(np.float32)) for x in (kf, vf))
        out = np.empty((B, H, q.shape[2], D), np.float32)
        lse = np.empty((B, H, q.shape[2]), np.float32)
        for (l0, n, g0) in segs:
            o_seg, l_seg = oracle.attention_fwd(np.ascontiguousarray(qn[:, :, l0:l0 + n]), kf, vf, D ** -0.5, cfg["causal"], q_off=g0, k_off=0)
            out[:, :, l0:l0 + n], lse[:, :, l0:l0 + n] = o_seg, l_seg
        good = bench.check_parity(rig, cfg, seed, q, torch.from_numpy(out), torch.from_numpy(lse), segs, 2, 24)
        bad_out = out.copy()
        if rank == 1:
            bad_out[:, :, 0, :] += 0.01          # row 0 is always among the sampled rows
        bad = bench.check_parity(rig, cfg, seed, q, torch.from_numpy(bad_out), torch.from_numpy(lse), segs, 2, 24)
        nan_out = out.copy()
        if rank == 0:
            nan_out[0, 0, -1, :] = np.nan        # a row nobody wrote
        unwritten = bench.check_parity(rig, cfg, seed, q, torch.from_numpy(nan_out), torch.from_numpy(lse), segs, 2, 24)
        res[name] = {"good": good["ok"], "good_err": good["max_abs_o"], "bad": bad["ok"], "bad_err": bad["max_abs_o"],
                     "unwritten": unwritten["ok"], "unwritten_flag": unwritten["unwritten_outputs"], "rows": good["rows"],
                     "seqlens": seqlens}
    import json
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


def test_parity_check_on_gloo_ranks(tmp_path):
    import json
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    per_rank = [json.load(open(os.path.join(str(tmp_path), f"rank{r}.json"))) for r in range(world)]
    for name in CASES:
        for r in range(world):
            got = per_rank[r][name]
            assert got["good"] is True and got["good_err"] <= 1e-6, (name, r, got)
            assert got["bad"] is False and got["bad_err"] >= 5e-3, (name, r, got)      # rank 1's wrong row fails rank 0 too
            assert got["unwritten"] is False and got["unwritten_flag"] is True, (name, r, got)
            assert got["rows"] >= 2 * 20
        assert per_rank[0][name] == per_rank[1][name]                                  # every rank reports the reduced result


def test_bench_config_table_is_consistent():
    import bench
    for name, cfg in bench.CONFIGS.items():
        sl = cfg.get("seqlens")
        assert sl is None or (len(sl) == cfg["world"] and sum(sl) == cfg["S"]), name
        assert cfg["S"] % cfg["world"] == 0 or sl is not None, name
        if cfg.get("zigzag"):
            assert cfg["causal"] and (cfg["S"] // cfg["world"]) % 2 == 0, name
    # BASELINE.json's five configurations are all there, on the GPU counts it names
    assert [bench.CONFIGS[n]["world"] for n in ("c1", "c2", "c3", "c4", "c5")] == [1, 2, 4, 8, 8]
    assert bench.config_flops(bench.CONFIGS["c1"]) == 4.0 * 64 * 8 * 1024 * 1024
    c4 = bench.CONFIGS["c4"]
    assert bench.config_flops(c4) == 4.0 * 128 * 32 * (131072 * 131073 / 2)


def test_reference_arm_under_a_two_process_launcher():
    """`bench.py --impl reference` launched like the multi-GPU arm (torchrun, two processes, which exports
    OMP_NUM_THREADS=1): rank 0 alone prints the line, it uses every host core all the same, labels the workload of
    that GPU count, and carries the same `config` object as the GPU arm would."""
    import json
    import subprocess
    import bench
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
           "--steps", "1", "--warmup", "0"]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, lines                       # the other rank exits without a line
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["gpu_launches"] == 0
    assert d["config"] == bench.workload_config(2) and "total seq 16384" in d["config"]["workload"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    assert d["e2e"]["value"] == d["value"] > 0 and d["e2e"]["h2d_bytes_per_step"] == 0
