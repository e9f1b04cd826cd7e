#!/usr/bin/env python
"""Benchmark of the ring-attention forward (the one hot path of this repository).

    python bench.py --gpus N --steps K --warmup W            # this implementation (CUDA, sm_100a)
    python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference path

For N > 1 it is launched one process per GPU (torchrun); ranks shard the sequence, exchange K/V over
NVLink and rank 0 prints ONE JSON line.  A "step" is one ring-attention forward over every rank's shard.

Headline workload (config.workload): configs[1] of BASELINE.json at one GPU -- batch 2, 16 heads, head_dim
128, fp16, non-causal, 8192 sequence rows per GPU; with N GPUs the total sequence is 8192 * N (weak scaling:
rows per GPU fixed).  Inputs are seeded synthetic N(0,1) values; Q, K and V together are 192 MiB per GPU,
larger than the 126 MB L2, so no explicit L2 flush is needed between timed iterations.

Besides the timed headline the line carries, all measured outside the timed regions:
  parity    sampled rows of every rank's output against the fp64 CPU oracle over the full K/V (max over ranks);
            a failed check makes the run exit non-zero;
  configs   the BASELINE.json configurations that fit this GPU count (c1 at 1 GPU, c2 at 2, c3 at 4, c4
            contiguous and zig-zag and c5 at 8) plus uneven-shard and bf16 cases, each with throughput and parity;
  exchange  per-ring-step compute / wait / copy / exposed times, mean over forwards, max over ranks;
  exchange_nccl  the same forward with NCCL send/recv as the transport, per CTA cap (N > 1);
  k1_probes the block kernel alone in the situations a ring step puts it in.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

B, H, S_LOCAL, D = 2, 16, 8192, 128
SEED = 1234
METRIC = "attention_fwd_tflops"
UNIT = "TFLOP/s"
TOL_O_MAXABS, TOL_O_RELL2, TOL_LSE = 2e-3, 1e-3, 1e-4   # BASELINE.json's parity bar
NVLINK_MEASURED_GBS, NVLINK_NOMINAL_GBS = 770.0, 900.0   # per direction per GPU

# dram__bytes_read.sum + dram__bytes_write.sum of ONE block-kernel launch at the bench shape, from an ncu capture
# of this kernel (201.7 MB read + 100.2 MB written).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 301.9e6

# BASELINE.json configurations and the extra cases, by the GPU count they run on.
#   S: total sequence; seqlens: rows per rank when the shards differ (sum = S)
CONFIGS = {
    "c1": dict(world=1, B=1, H=8, S=1024, D=64, causal=False, gain=1.0, heads=2, rows=48, reps=50),
    "d64_b4_h16_s4096": dict(world=1, B=4, H=16, S=4096, D=64, causal=False, gain=1.0, heads=2, rows=32, reps=20),
    "bf16_b2_h8_s2048_causal": dict(world=1, B=2, H=8, S=2048, D=128, causal=True, gain=1.0, heads=2, rows=32, reps=20, bf16=True),
    "c2": dict(world=2, B=2, H=16, S=8192, D=128, causal=False, gain=1.0, heads=3, rows=64, reps=10),
    "uneven2": dict(world=2, B=1, H=4, S=4096 + 2176, D=128, causal=True, gain=1.0, heads=2, rows=48, reps=5, seqlens=[4096, 2176]),
    "bf16_2": dict(world=2, B=1, H=8, S=4096, D=128, causal=True, gain=1.0, heads=2, rows=48, reps=5, bf16=True),
    "c3": dict(world=4, B=1, H=32, S=32768, D=128, causal=False, gain=0.5, heads=3, rows=64, reps=5),
    "uneven4": dict(world=4, B=1, H=4, S=4096 + 2176 + 8192 + 1152, D=128, causal=False, gain=1.0, heads=2, rows=48, reps=5,
                    seqlens=[4096, 2176, 8192, 1152]),
    "c4": dict(world=8, B=1, H=32, S=131072, D=128, causal=True, gain=1.0, heads=2, rows=48, reps=3),
    "c4_zigzag": dict(world=8, B=1, H=32, S=131072, D=128, causal=True, gain=1.0, heads=2, rows=48, reps=3, zigzag=True),
    "c5": dict(world=8, B=1, H=8, S=1048576, D=128, causal=False, gain=1.0, heads=1, rows=24, reps=3),
    "uneven8": dict(world=8, B=1, H=4, S=2 * (4096 + 2176 + 3200 + 1152), D=64, causal=True, gain=1.0, heads=2, rows=32, reps=3,
                    seqlens=[4096, 2176, 3200, 1152, 1152, 3200, 2176, 4096]),
}


def flops_per_rank(world: int) -> float:
    """4 * D * B * H * (#unmasked (q, k) pairs) for one rank: its S_LOCAL rows against all keys."""
    return 4.0 * D * B * H * S_LOCAL * (S_LOCAL * world)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"tflops": float(p["bf16_tflops"]), "tflops_sustained": float(p.get("bf16_tflops_sustained", 0.0)),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def workload_name(world: int) -> str:
    return (f"BASELINE configs[1] shape per GPU: batch {B}, heads {H}, head_dim {D}, fp16, non-causal, "
            f"{S_LOCAL} rows/GPU, total seq {S_LOCAL * world}")


def workload_config(world: int) -> dict:
    """The `config` object of the JSON line: identical for the GPU arm and the reference arm at the same N."""
    return {"workload": workload_name(world), "batch": B, "heads": H, "seq_local": S_LOCAL, "seq_total": S_LOCAL * world,
            "head_dim": D, "causal": False, "seed": SEED,
            "parallelism": f"ring{world} (sequence sharded over {world} GPU(s), double-buffered K/V exchange on a side stream)",
            "l2": "inputs (192 MiB of Q,K,V per GPU) exceed the 126 MB L2; no flush between iterations"}


class ClockSampler:
    """SM clock and throttle-reason samples taken every 2 ms through NVML while the timed region runs
    (reads only; nothing on the GPU is changed)."""
    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = None
        self._thread = None
        self.error = None

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # no NVML: report that instead of a clock
            self.error = f"NVML unavailable: {e}"
            return
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                    for name, bit in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception as e:
                    self.error = str(e)
                    return
                time.sleep(0.002)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.error:
            out["note"] = self.error
        return out


# ------------------------------------------------------------------------------------------ CPU arm
def time_cpu_port(target_s: float, world: int = 1):
    """Times the CPU restatement of the reference path (oracle port, fp32 accumulate, OpenMP on every
    host core) on a bounded sample of the bench workload: query rows of the first heads of batch 0 against
    all 8192 * world keys of their head, sized from a short probe to about `target_s` seconds.
    Returns (tflops, cores, sample description, seconds)."""
    from oracle import oracle
    from ringattention_b200 import synthetic
    cores = oracle.set_num_threads(os.cpu_count() or 1)   # launchers export OMP_NUM_THREADS=1 to their workers
    S = S_LOCAL * world
    scale = D ** -0.5

    def head(which, h, rows):
        return synthetic.make_head(which, SEED, H, D, 0, h, 0, rows)

    q0, k0, v0 = head("q", 0, S_LOCAL)[None, None], head("k", 0, S)[None, None], head("v", 0, S)[None, None]
    probe = 128
    t0 = time.perf_counter()
    oracle.attention_fwd(np.ascontiguousarray(q0[:, :, :probe]), k0, v0, scale, accum="f32")
    per_row = max(time.perf_counter() - t0, 1e-4) / probe
    rows_total = max(probe, int(target_s / per_row))
    n_heads = int(min(H, max(1, rows_total // S_LOCAL)))
    rows = S_LOCAL if rows_total >= S_LOCAL else max(128, rows_total // 128 * 128)
    q = np.stack([head("q", h, rows) for h in range(n_heads)])[None]
    k = np.stack([head("k", h, S) for h in range(n_heads)])[None]
    v = np.stack([head("v", h, S) for h in range(n_heads)])[None]
    t0 = time.perf_counter()
    oracle.attention_fwd(q, k, v, scale, accum="f32")
    dt = time.perf_counter() - t0
    fl = 4.0 * D * n_heads * rows * S
    return fl / dt / 1e12, cores, (f"first {rows} query rows of heads 0..{n_heads - 1} of batch 0 x all {S} keys of each head, "
                                   f"fp32 accumulate"), dt


def run_reference_arm(args, rank: int):
    """--impl reference: the reference's CPU implementation of the path.  The reference itself has no CPU
    attention and its CUDA source does not compile, so this is the oracle port (kind = "port").  Under a
    multi-process launcher rank 0 alone runs it, on all host cores."""
    if rank != 0:
        return
    vals, secs = [], []
    cores, sample = 1, ""
    per_step = max(2.0, min(12.0, 120.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        tf, cores, sample, dt = time_cpu_port(per_step, args.gpus)
        if i >= args.warmup:
            vals.append(tf); secs.append(dt)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.mean(secs)) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "note": "each step is a bounded sample of the workload; value = sample flops / sample time (no extrapolation)",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm helpers
class Rig:
    """What every part of the GPU arm needs: device, rank, the process group (or None)."""

    def __init__(self, torch, dist, dev, rank, world):
        self.torch, self.dist, self.dev, self.rank, self.world = torch, dist, dev, rank, world
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        """Element-wise max / min / sum of a list of floats over the ranks."""
        if self.dist is None:
            return [float(x) for x in values]
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        ops = {"max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN, "sum": self.dist.ReduceOp.SUM}
        self.dist.all_reduce(t, op=ops[op])
        return [float(x) for x in t.tolist()]

    def timed(self, fn, steps):
        """K calls of fn bracketed by barrier + synchronize; returns (ms of the slowest rank, this rank's per-step ms)."""
        self.barrier()
        marks = [self.torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record(self.stream)
        for i in range(steps):
            fn()
            marks[i + 1].record(self.stream)
        marks[-1].synchronize()
        self.barrier()
        ms = self.reduce([marks[0].elapsed_time(marks[-1])], "max")[0]
        return ms, [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]


def make_rank_inputs(rig: Rig, cfg: dict, seed: int):
    """This rank's shard of the seeded global tensors for configuration `cfg`.
    Returns (q, k, v device tensors, segments, seqlens): segments = [(local_start, rows, global_start)]."""
    from ringattention_b200 import synthetic
    torch = rig.torch
    world, r = rig.world, rig.rank
    Bc, Hc, S, Dc, gain = cfg["B"], cfg["H"], cfg["S"], cfg["D"], cfg["gain"]
    seqlens = cfg.get("seqlens") or [S // world] * world
    assert len(seqlens) == world and sum(seqlens) == S
    Sl = seqlens[r]
    if cfg.get("zigzag"):
        ch = Sl // 2
        g0, g1 = r * ch, (2 * world - 1 - r) * ch
        parts = [synthetic.make_qkv(seed, Bc, Hc, Dc, g0, ch, gain), synthetic.make_qkv(seed, Bc, Hc, Dc, g1, ch, gain)]
        host = [np.concatenate([parts[0][i], parts[1][i]], axis=2) for i in range(3)]
        segs = [(0, ch, g0), (ch, ch, g1)]
    else:
        g0 = sum(seqlens[:r])
        host = list(synthetic.make_qkv(seed, Bc, Hc, Dc, g0, Sl, gain))
        segs = [(0, Sl, g0)]
    q, k, v = (torch.from_numpy(x).to(rig.dev) for x in host)
    if cfg.get("bf16"):
        q, k, v = (x.float().to(torch.bfloat16) for x in (q, k, v))   # exact widening, then round to nearest even
    return q, k, v, segs, seqlens


def check_parity(rig: Rig, cfg: dict, seed: int, q_dev, out_dev, lse_dev, segs, n_heads: int, n_rows: int) -> dict:
    """Seeded sample rows of THIS rank's output against the fp64 CPU oracle evaluated over the full global
    K/V of the sampled heads (regenerated from the seed, never read back from a GPU); errors max-reduced
    over ranks.  This is the check the multi-GPU exchange is held to: a stale or misplaced shard shows here."""
    from oracle import oracle
    from ringattention_b200 import synthetic
    torch = rig.torch
    Bc, Hc, S, Dc, gain, causal = cfg["B"], cfg["H"], cfg["S"], cfg["D"], cfg["gain"], cfg["causal"]
    bf16 = bool(cfg.get("bf16"))
    scale = Dc ** -0.5
    Sl = q_dev.shape[2]
    rng = np.random.Generator(np.random.Philox(key=np.array([seed, rig.rank], dtype=np.uint64)))
    heads = sorted({(int(rng.integers(0, Bc)), int(rng.integers(0, Hc))) for _ in range(n_heads)})
    o_host, l_host = out_dev.cpu().numpy(), lse_dev.cpu().numpy()
    unwritten = bool(np.isnan(o_host).any() or np.isnan(l_host).any())
    err_o = err_l = num = den = 0.0
    nrows = 0
    t0 = time.time()

    def as_oracle_input(x16: np.ndarray) -> np.ndarray:
        return oracle.to_bf16_bits(x16.astype(np.float32)) if bf16 else x16

    for (b, h) in heads:
        idx = np.unique(np.concatenate([[0, Sl - 1, Sl // 2, max(Sl // 2 - 1, 0)], rng.integers(0, Sl, n_rows)])).astype(np.int64)
        kf = as_oracle_input(synthetic.make_head("k", seed, Hc, Dc, b, h, 0, S, gain))[None, None]
        vf = as_oracle_input(synthetic.make_head("v", seed, Hc, Dc, b, h, 0, S, gain))[None, None]
        qh = q_dev[b, h].contiguous()
        qh = (qh.view(torch.int16).cpu().numpy().view(np.uint16) if bf16 else qh.cpu().numpy())[None, None]
        rows = np.stack([np.zeros_like(idx), np.zeros_like(idx), idx], axis=1)
        want_o = np.empty((len(idx), Dc), np.float32)
        want_l = np.empty(len(idx), np.float32)
        for (l0, n, g0) in segs:   # global index of local row i of a segment: g0 + (i - l0)
            sel = (idx >= l0) & (idx < l0 + n)
            if sel.any():
                want_o[sel], want_l[sel] = oracle.attention_rows(qh, kf, vf, rows[sel], scale, causal, q_off=g0 - l0, k_off=0)
        got_o, got_l = o_host[b, h, idx], l_host[b, h, idx]
        with np.errstate(invalid="ignore"):
            err_o = max(err_o, float(np.nanmax(np.abs(got_o - want_o))))
            err_l = max(err_l, float(np.nanmax(np.abs(got_l - want_l))))
        num += float(((got_o - want_o) ** 2).sum()); den += float((want_o ** 2).sum())
        nrows += len(idx)
    mx = rig.reduce([err_o, err_l, float(unwritten), time.time() - t0], "max")
    sm = rig.reduce([num, den, nrows], "sum")
    rel = float(np.sqrt(sm[0] / max(sm[1], 1e-300)))
    # bf16 inputs: P is rounded to 8 significant bits before P V (relative error <= 2^-9 per element, row sums
    # unrounded), so |dO| <= 2^-9 * max|v| and rel-L2 <= 2^-9; the fp16 bar is BASELINE.json's.
    tol_o = max(TOL_O_MAXABS, 2.0 ** -9 * 6.0 * gain) if bf16 else TOL_O_MAXABS   # |N(0,1)| draws stay below 6
    tol_rel = 2.0 ** -9 if bf16 else TOL_O_RELL2
    ok = bool(mx[2] == 0.0 and mx[0] <= tol_o and rel <= tol_rel and mx[1] <= TOL_LSE)
    return {"max_abs_o": mx[0], "rel_l2_o": rel, "max_abs_lse": mx[1], "rows": int(sm[2]), "unwritten_outputs": bool(mx[2]),
            "tol": {"max_abs_o": tol_o, "rel_l2_o": tol_rel, "max_abs_lse": TOL_LSE},
            "against": "fp64 CPU oracle over the full global K/V of the sampled heads", "oracle_s": mx[3], "ok": ok}


def exchange_stats(rig: Rig, ctx, fwd, n_fwd: int, kv_bytes_per_step: float) -> dict:
    """Per-ring-step timings from the context's events, over n_fwd untimed forwards (each followed by a
    synchronize so that its events can be read): mean over the forwards, max over the ranks.  The exchange is
    split into the wait for its go-ahead and the copy itself; achieved GB/s is bytes / copy time."""
    P = rig.world
    comp = np.zeros((n_fwd, P)); wait = np.zeros((n_fwd, P)); copy = np.zeros((n_fwd, P)); expo = np.zeros((n_fwd, P))
    for i in range(n_fwd):
        rig.barrier()
        fwd()
        ctx.synchronize()
        c, _, e = ctx.timings()
        w, cp = ctx.exchange_timings()
        comp[i], expo[i], wait[i], copy[i] = c, e, w, cp
    flat = rig.reduce(list(comp.ravel()) + list(expo.ravel()) + list(wait.ravel()) + list(copy.ravel()), "max")
    n = n_fwd * P
    comp_m, expo_m, wait_m, copy_m = (np.array(flat[i * n:(i + 1) * n]).reshape(n_fwd, P) for i in range(4))
    frac_mine = expo.sum(axis=1) / np.maximum(comp.sum(axis=1) + expo.sum(axis=1), 1e-9)   # this rank, per forward
    frac_max = rig.reduce(list(frac_mine), "max")
    copy_steps = copy_m[:, :P - 1] if P > 1 else copy_m[:, :0]
    copy_mean = float(copy_steps.mean()) if copy_steps.size else 0.0
    return {
        "forwards_sampled": n_fwd, "aggregation": "mean over forwards of the max over ranks, per ring step",
        "compute_ms_per_ring_step": comp_m.mean(axis=0).tolist(),
        "exposed_ms_per_ring_step": expo_m.mean(axis=0).tolist(),
        "exchange_wait_ms_per_ring_step": wait_m.mean(axis=0).tolist(),
        "exchange_copy_ms_per_ring_step": copy_m.mean(axis=0).tolist(),
        "compute_ms_per_ring_step_rank0": comp.mean(axis=0).tolist(),
        "exposed_frac": float(np.mean(frac_max)), "exposed_frac_worst_forward": float(np.max(frac_max)),
        "kv_bytes_per_ring_step": kv_bytes_per_step,
        "achieved_gbs": (kv_bytes_per_step / (copy_mean * 1e-3) / 1e9) if copy_mean > 0 else None,
        "nvlink_floor_ms": {"at_measured_770_gbs": kv_bytes_per_step / (NVLINK_MEASURED_GBS * 1e9) * 1e3,
                            "at_nominal_900_gbs": kv_bytes_per_step / (NVLINK_NOMINAL_GBS * 1e9) * 1e3},
    }


def config_flops(cfg: dict) -> float:
    S = cfg["S"]
    pairs = S * (S + 1) / 2.0 if cfg["causal"] else float(S) * S
    return 4.0 * cfg["D"] * cfg["B"] * cfg["H"] * pairs


def run_config(rig: Rig, ra, ctx, name: str, cfg: dict) -> dict:
    """One BASELINE.json configuration (or extra case) on this GPU count: one warm-up forward, `reps` timed forwards
    (each bracketed by a barrier; time of the slowest rank), per-rank busy time, exposed exchange, parity."""
    torch = rig.torch
    seed = SEED + 17
    t0 = time.time()
    q, k, v, segs, seqlens = make_rank_inputs(rig, cfg, seed)
    gen_s = time.time() - t0
    Bc, Hc, Dc = cfg["B"], cfg["H"], cfg["D"]
    Sl = seqlens[rig.rank]
    out = torch.full((Bc, Hc, Sl, Dc), float("nan"), device=rig.dev)
    lse = torch.full((Bc, Hc, Sl), float("nan"), device=rig.dev)
    scale = Dc ** -0.5
    ctx.set_option(ra.RING_OPT_CAUSAL_ZIGZAG, int(bool(cfg.get("zigzag"))))

    def fwd():
        ctx.forward(q, k, v, out, lse, causal=cfg["causal"], softmax_scale=scale, seqlens=seqlens)

    fwd()
    ctx.synchronize()
    reps = max(3, int(cfg.get("reps", 3)))
    ms, _ = rig.timed(fwd, reps)
    ctx.synchronize()
    ms_fwd = ms / reps
    xs = exchange_stats(rig, ctx, fwd, 2, 2.0 * Bc * Hc * max(seqlens) * Dc * 2) if rig.world > 1 else None
    # busy time of this rank (sum of its block-kernel time over the ring steps) from one more recorded forward
    fwd(); ctx.synchronize()
    comp, _, _ = ctx.timings()
    busy_ms = float(sum(comp))
    S = cfg["S"]
    g0s = [g for (_, _, g) in segs]
    if cfg["causal"]:   # row with global index g sees g + 1 keys
        pairs_mine = sum(n * g + n * (n + 1) / 2.0 for (_, n, g) in segs)
    else:
        pairs_mine = float(Sl) * S
    my_tflops_busy = 4.0 * Dc * Bc * Hc * pairs_mine / max(busy_ms * 1e-3, 1e-9) / 1e12
    busy = rig.reduce([my_tflops_busy], "min") + rig.reduce([my_tflops_busy], "max")
    # The forward lasts as long as its busiest rank (under a contiguous causal mask the last one): what the exchange
    # costs is the part of the forward that rank did not spend in its kernels.  The max over ranks of a rank's own
    # exposed fraction (exposed_frac below) also counts lightly loaded ranks waiting for work that delays nobody.
    busy_ms_max = rig.reduce([busy_ms], "max")[0]
    par = check_parity(rig, cfg, seed, q, out, lse, segs, cfg["heads"], cfg["rows"])
    ctx.set_option(ra.RING_OPT_CAUSAL_ZIGZAG, 0)
    res = {"shape": {k2: cfg[k2] for k2 in ("B", "H", "S", "D", "causal", "gain")}, "world": rig.world,
           "dtype": "bf16" if cfg.get("bf16") else "f16", "sharding": "zigzag" if cfg.get("zigzag") else "contiguous",
           "seqlens": seqlens if cfg.get("seqlens") else None,
           "forwards_timed": reps, "ms_per_forward": ms_fwd,
           "tflops_per_gpu": config_flops(cfg) / (ms_fwd * 1e-3) / 1e12 / rig.world,
           "busy_tflops_per_rank_min_max": busy,
           "busiest_rank_kernel_ms": busy_ms_max,
           "exposed_frac_busiest_rank": max(0.0, 1.0 - busy_ms_max / ms_fwd) if rig.world > 1 else 0.0,
           "exposed_frac": xs["exposed_frac"] if xs else 0.0,
           "exchange": xs, "parity": par, "gen_s": gen_s, "first_global_rows_rank0": g0s}
    del q, k, v, out, lse
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------ GPU arm
def run_gpu_arm(args, rank: int, local_rank: int, world: int):
    import torch
    import ringattention_b200 as ra
    from ringattention_b200 import synthetic

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for this path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    rig = Rig(torch, dist, dev, rank, world)
    stream = rig.stream
    scale = D ** -0.5

    # ---- inputs: this rank's rows of the global seeded tensors, in pinned host memory and on the device
    hq, hk, hv = (torch.from_numpy(x).pin_memory() for x in synthetic.make_qkv(SEED, B, H, D, rank * S_LOCAL, S_LOCAL))
    q, k, v = (x.to(dev) for x in (hq, hk, hv))
    out = torch.full((B, H, S_LOCAL, D), float("nan"), dtype=torch.float32, device=dev)
    lse = torch.full((B, H, S_LOCAL), float("nan"), dtype=torch.float32, device=dev)
    h_out = torch.empty(out.shape, dtype=torch.float32).pin_memory()
    h_lse = torch.empty(lse.shape, dtype=torch.float32).pin_memory()
    reps = 50
    k1_flops = 4.0 * D * B * H * S_LOCAL * S_LOCAL

    def k1_time(merge=False, side_copies=None, n=reps):
        """Block kernel alone (one shard against one shard): ms per launch by CUDA events over n launches on the
        launching stream.  side_copies: (stream, src, dst) -> two device-to-device copies are queued per launch."""
        for _ in range(3):
            ra.attention_block_fwd(q, k, v, out, lse, softmax_scale=scale, merge=merge)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            if side_copies is not None:
                st, a, b2 = side_copies
                with torch.cuda.stream(st):
                    b2.copy_(a, non_blocking=True)
                    a.copy_(b2, non_blocking=True)
            ra.attention_block_fwd(q, k, v, out, lse, softmax_scale=scale, merge=merge)
        e1.record(stream)
        e1.synchronize()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    # ---- the block kernel before any ring step or communicator exists on this GPU (power-steady: ~400 ms of it first)
    for _ in range(3):
        ra.attention_block_fwd(q, k, v, out, lse, softmax_scale=scale)
    torch.cuda.synchronize()
    k1_time(n=int(max(50, args.prewarm_ms)))   # ~1 ms per launch
    k1_before_ms = k1_time()

    ctx = ra.RingContext.from_torch_distributed() if world > 1 else ra.RingContext.create(0, 1, None)
    ctx.set_option(ra.RING_OPT_RECORD_TIMINGS, 1)
    if args.merge_mode is not None:
        ctx.set_option(ra.RING_OPT_MERGE_MODE, args.merge_mode)
    if world > 1 and args.transport != "default":
        ctx.set_option(ra.RING_OPT_TRANSPORT, ra.RING_TRANSPORT_NCCL if args.transport == "nccl" else ra.RING_TRANSPORT_PEER_COPY)
    transport = "none (one rank)"
    if world > 1:
        transport = ("copy-engine pushes into IPC-shared receive buffers" if ctx.get_option(ra.RING_OPT_TRANSPORT) == ra.RING_TRANSPORT_PEER_COPY
                     else "NCCL send/recv")

    def step_resident():
        ctx.forward(q, k, v, out, lse, softmax_scale=scale)

    def step_e2e():
        # the public host-buffer call: pinned Q, K, V in, pinned O, LSE out, copies inside the timed region
        ctx.forward_host(hq, hk, hv, h_out, h_lse, chunks=args.e2e_chunks, softmax_scale=scale)

    for _ in range(max(args.warmup, 3)):
        step_resident()
    ctx.synchronize()
    # Power-steady state: a B200 runs a short burst at 1965 MHz and settles near 1.5 GHz under its 1 kW cap after
    # about half a second of this kernel.  With N GPUs a step is N times longer, so without this phase the
    # N = 1 line would be a burst number and the N = 8 line a sustained one.  Untimed; same count on every rank.
    probe_ms = rig.timed(step_resident, 3)[0] / 3
    n_pre = int(min(4000, max(0, args.prewarm_ms / max(probe_ms, 1e-3))))
    for _ in range(n_pre):
        step_resident()
    ctx.synchronize()

    # ---- the timed regions: `regions` times EXACTLY `steps` forwards, each region bracketed by barrier + synchronize
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ra.kernel_launch_count()
    region_ms, steps_ms = [], []
    for _ in range(max(1, args.regions)):
        ms, mine = rig.timed(step_resident, args.steps)
        region_ms.append(ms)
        steps_ms.extend(mine)
    launches = (ra.kernel_launch_count() - launches0) // max(1, args.regions)
    ctx.synchronize()  # also checks the device status word
    clocks = sampler.stop() if rank == 0 else None
    total_ms = statistics.median(region_ms)

    # ---- parity of the headline forward: the output the timed steps left behind, against the fp64 oracle
    head_cfg = dict(B=B, H=H, S=S_LOCAL * world, D=D, causal=False, gain=1.0)
    parity = check_parity(rig, head_cfg, SEED, q, out, lse, [(0, S_LOCAL, rank * S_LOCAL)], 2, 32)

    # ---- per-ring-step compute / wait / copy / exposed (untimed forwards)
    kv_bytes = 2.0 * B * H * S_LOCAL * D * 2
    exchange = exchange_stats(rig, ctx, step_resident, min(10, max(3, args.steps)), kv_bytes)
    exchange["kv_transport"] = transport

    # ---- dominant kernel alone, right after the timed region so that it sees the same power-steady clocks; then
    # the situations a ring step puts it in (folding into a partial; copies running beside it), interleaved with the
    # plain form in short batches so that drifting clocks under the power cap hit every variant alike
    for _ in range(5):
        step_resident()
    k1_ms = k1_time()
    side = torch.cuda.Stream(priority=-1)
    buf_a = torch.empty(int(kv_bytes), dtype=torch.uint8, device=dev)
    buf_b = torch.empty_like(buf_a)
    probe = {"plain": [], "merge": [], "copies": []}
    probe_mhz = {"plain": [], "merge": [], "copies": []}

    def probed(name, **kw):
        # SM clock sampled while the batch runs: time x clock tells a slower kernel (more clocks) from a lower clock
        # (the power cap answering extra memory traffic)
        smp = ClockSampler(local_rank)
        if rank == 0:
            smp.start()
        probe[name].append(k1_time(n=40, **kw))
        if rank == 0:
            mhz = smp.stop().get("sm_mhz")
            if mhz:
                probe_mhz[name].append(mhz)

    for _ in range(4):
        probed("plain")
        probed("merge", merge=True)
        probed("copies", side_copies=(side, buf_a, buf_b))
    del buf_a, buf_b
    # the library GEMM the roofline's denominator was measured with, under the same power-steady protocol, same run
    ga = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    gb = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    gc = torch.empty(8192, 8192, device=dev, dtype=torch.bfloat16)
    for _ in range(3):
        torch.matmul(ga, gb, out=gc)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(300):                      # ~0.25 s of it first: the power-steady state of THIS kernel
        torch.matmul(ga, gb, out=gc)
    e0.record(stream)
    for _ in range(reps):
        torch.matmul(ga, gb, out=gc)
    e1.record(stream)
    e1.synchronize()
    cublas_sustained_tflops = 2.0 * 8192 ** 3 / (e0.elapsed_time(e1) / reps * 1e-3) / 1e12
    # and both in the protocol the burst peak was taken with: after an idle pause, best of 10 single launches
    def burst(fn):
        torch.cuda.synchronize()
        time.sleep(1.0)
        best = 1e9
        for _ in range(10):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream); fn(); a1.record(stream); a1.synchronize()
            best = min(best, a0.elapsed_time(a1))
        return best
    k1_burst_ms = burst(lambda: ra.attention_block_fwd(q, k, v, out, lse, softmax_scale=scale))
    cublas_burst_tflops = 2.0 * 8192 ** 3 / (burst(lambda: torch.matmul(ga, gb, out=gc)) * 1e-3) / 1e12
    del ga, gb, gc
    assert ra.device_status() == 0

    # ---- end to end: host buffers in, host buffers out, every step
    for _ in range(2):
        step_e2e()
    e2e_ms, _ = rig.timed(step_e2e, args.steps)
    ctx.synchronize()
    e2e_cfg_ok = check_parity(rig, head_cfg, SEED, q, h_out.to(dev), h_lse.to(dev), [(0, S_LOCAL, rank * S_LOCAL)], 1, 16)

    # ---- merge kernel alone (HBM bound), for the record
    o2, l2 = torch.empty_like(out), torch.empty_like(lse)
    ra.attention_block_fwd(q, k, v, o2, l2, softmax_scale=scale)
    for _ in range(3):
        ra.lse_merge(out, lse, o2, l2)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        ra.lse_merge(out, lse, o2, l2)
    e1.record(stream)
    e1.synchronize()
    k2_ms = e0.elapsed_time(e1) / reps
    del o2, l2

    # ---- BASELINE.json configurations that belong to this GPU count (+ uneven shards, bf16)
    configs = {}
    if args.configs != "none":
        wanted = [n for n, c in CONFIGS.items() if c["world"] == world] if args.configs == "auto" else args.configs.split(",")
        for name in wanted:
            if name not in CONFIGS or CONFIGS[name]["world"] != world:
                continue
            try:
                configs[name] = run_config(rig, ra, ctx, name, CONFIGS[name])
            except Exception as e:  # a failing case must not cost the whole line; it is reported as failed
                configs[name] = {"error": f"{type(e).__name__}: {e}", "parity": {"ok": False}}

    # ---- the same forward with NCCL send/recv as the transport (what BASELINE.json names), per CTA cap
    exchange_nccl = None
    if world > 1 and args.nccl_ctas != "none" and transport.startswith("copy-engine"):
        exchange_nccl = {}
        for cap in [int(x) for x in args.nccl_ctas.split(",")]:
            os.environ["RING_TRANSPORT"] = "nccl"
            os.environ["RING_NCCL_MAX_CTAS"] = str(cap)
            try:
                c2 = ra.RingContext.from_torch_distributed()
                c2.set_option(ra.RING_OPT_RECORD_TIMINGS, 1)

                def step_nccl():
                    c2.forward(q, k, v, out, lse, softmax_scale=scale)

                for _ in range(3):
                    step_nccl()
                c2.synchronize()
                ms, _ = rig.timed(step_nccl, args.steps)
                c2.synchronize()
                xs = exchange_stats(rig, c2, step_nccl, 3, kv_bytes)
                par = check_parity(rig, head_cfg, SEED, q, out, lse, [(0, S_LOCAL, rank * S_LOCAL)], 1, 16)
                exchange_nccl[f"max_ctas_{cap}"] = {
                    "per_gpu_tflops": flops_per_rank(world) / (ms / args.steps * 1e-3) / 1e12, "ms_per_step": ms / args.steps,
                    "exposed_frac": xs["exposed_frac"], "compute_ms_per_ring_step": xs["compute_ms_per_ring_step"],
                    "exposed_ms_per_ring_step": xs["exposed_ms_per_ring_step"],
                    "exchange_copy_ms_per_ring_step": xs["exchange_copy_ms_per_ring_step"], "parity_ok": par["ok"]}
                c2.destroy()
            except Exception as e:
                exchange_nccl[f"max_ctas_{cap}"] = {"error": f"{type(e).__name__}: {e}"}
            finally:
                os.environ.pop("RING_TRANSPORT", None)
                os.environ.pop("RING_NCCL_MAX_CTAS", None)

    all_ok = parity["ok"] and e2e_cfg_ok["ok"] and all(c.get("parity", {}).get("ok", False) for c in configs.values())
    if rank == 0:
        peaks = load_peaks()
        ms_per_step = total_ms / args.steps
        job_flops = flops_per_rank(world) * world
        value = job_flops / (ms_per_step * 1e-3) / 1e12
        region_values = [job_flops / (m / args.steps * 1e-3) / 1e12 for m in region_ms]
        e2e_value = job_flops / (e2e_ms / args.steps * 1e-3) / 1e12
        k1_tflops = k1_flops / (k1_ms * 1e-3) / 1e12
        k2_bytes = (3 * D + 3) * 4.0 * B * H * S_LOCAL
        cpu_tf, cores, sample, _ = time_cpu_port(12.0) if world == 1 else (None, None, None, None)
        mhz = (clocks or {}).get("sm_mhz")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world),
            "timing": {"regions": len(region_ms), "steps_per_region": args.steps,
                       "value_is": "median over the regions; each region is exactly `steps` forwards between barrier + synchronize, max over ranks",
                       "region_values": region_values, "spread_frac": (max(region_values) - min(region_values)) / value,
                       "ms_per_step_median_rank0": statistics.median(steps_ms), "ms_per_step_min_rank0": min(steps_ms),
                       "prewarm": f"{n_pre} untimed steps (~{args.prewarm_ms:.0f} ms) before the timed regions, to reach the power-capped steady clocks",
                       "ms_per_step_x_sm_ghz": (ms_per_step * mhz / 1e3) if mhz else None},
            "run": {"kv_transport": transport, "merge_mode": "separate kernel" if args.merge_mode == 0 else "fused epilogue"},
            "per_gpu_tflops": value / world,
            "parity": parity,
            "roofline": {"bound": "tensor", "kernel": "ring_block_attention_kernel<128,256,128,12,half>",
                         "achieved": k1_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": k1_tflops / peaks["tflops"],
                         "peak_source": peaks["source"] + " (cuBLAS bf16 burst; kernel timed in the power-steady state)",
                         "frac_of_sustained_peak": (k1_tflops / peaks["tflops_sustained"]) if peaks["tflops_sustained"] else None,
                         "frac_of_nominal_2250": k1_tflops / 2250.0,
                         "flops_per_launch": k1_flops, "ms_per_launch": k1_ms, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "same_run_reference": {
                             "what": "torch.matmul bf16 8192^3 (cuBLAS) timed in this run beside the kernel, on this GPU",
                             "power_steady": {"kernel_tflops": k1_tflops, "cublas_tflops": cublas_sustained_tflops,
                                              "ratio": k1_tflops / cublas_sustained_tflops},
                             "burst_after_1s_idle_best_of_10": {"kernel_tflops": k1_flops / (k1_burst_ms * 1e-3) / 1e12,
                                                                "cublas_tflops": cublas_burst_tflops,
                                                                "ratio": k1_flops / (k1_burst_ms * 1e-3) / 1e12 / cublas_burst_tflops}}},
            "k1_probes": {"what": "block kernel alone, ms per launch (rank 0), same shape as one ring step of the headline",
                          "before_any_ring_step": k1_before_ms, "after_timed_region": k1_ms,
                          "interleaved_batches_of_40": {"plain": probe["plain"], "folding_into_partial": probe["merge"],
                                                        "with_two_local_d2d_copies_of_a_kv_shard_per_launch_at_hbm_speed": probe["copies"]},
                          "median_ms": {kk: statistics.median(vv) for kk, vv in probe.items()},
                          "median_sm_mhz": {kk: (statistics.median(vv) if vv else None) for kk, vv in probe_mhz.items()},
                          "median_ms_x_sm_ghz": {kk: (statistics.median(probe[kk]) * statistics.median(vv) / 1e3 if vv else None)
                                                 for kk, vv in probe_mhz.items()}},
            "merge_kernel": {"bound": "hbm", "achieved": k2_bytes / (k2_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": k2_bytes / (k2_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "ms_per_launch": k2_ms},
            "exchange": exchange,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 3 * B * H * S_LOCAL * D * 2 * world,
                    "d2h_bytes_per_step": (B * H * S_LOCAL * D * 4 + B * H * S_LOCAL * 4) * world,
                    "parity_ok": e2e_cfg_ok["ok"]},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "configs": configs,
        }
        if exchange_nccl is not None:
            line["exchange_nccl"] = exchange_nccl
        if cpu_tf is not None:
            line["cpu_baseline"] = {"value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)

    ctx.destroy()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if not all_ok:
        raise SystemExit("bench.py: a parity check against the CPU oracle FAILED (see the parity objects of the line above)")


def run_block_only(spec: str):
    """--block-only B,H,Sq,Sk,D: a few launches of the block kernel alone on seeded inputs of that shape, one JSON line.
    A small, bounded case of the same kernel for profiler captures (RING_PAIR=1 in the environment selects the
    CTA-pair form)."""
    import torch
    import ringattention_b200 as ra
    from ringattention_b200 import synthetic
    Bc, Hc, Sq, Sk, Dc = (int(x) for x in spec.split(","))
    torch.cuda.set_device(0)
    q = torch.from_numpy(synthetic.make_shard("q", SEED, Bc, Hc, Dc, 0, Sq)).cuda()
    k = torch.from_numpy(synthetic.make_shard("k", SEED, Bc, Hc, Dc, 0, Sk)).cuda()
    v = torch.from_numpy(synthetic.make_shard("v", SEED, Bc, Hc, Dc, 0, Sk)).cuda()
    o = torch.empty((Bc, Hc, Sq, Dc), device="cuda")
    lse = torch.empty((Bc, Hc, Sq), device="cuda")
    for _ in range(3):
        ra.attention_block_fwd(q, k, v, o, lse)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 5
    e0.record()
    for _ in range(n):
        ra.attention_block_fwd(q, k, v, o, lse)
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1) / n
    assert ra.device_status() == 0
    fl = 4.0 * Dc * Bc * Hc * Sq * Sk
    print(json.dumps({"mode": "block-only", "shape": {"B": Bc, "H": Hc, "Sq": Sq, "Sk": Sk, "D": Dc}, "launches": 3 + n,
                      "form": "cta-pair" if os.environ.get("RING_PAIR", "0") not in ("", "0") and Dc == 128 else "one-cta",
                      "ms_per_launch": ms, "tflops": fl / (ms * 1e-3) / 1e12,
                      "hbm_bytes_algorithmic": 2.0 * Bc * Hc * (Sq + 2 * Sk) * Dc + 4.0 * Bc * Hc * Sq * (Dc + 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--regions", type=int, default=5, help="timed regions of `steps` forwards each; the value is their median")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="(batch, head) groups the host-buffer forward pipelines")
    ap.add_argument("--prewarm-ms", type=float, default=1500.0,
                    help="untimed forwards before the timed regions: a B200 needs about half a second of this kernel, from idle, before "
                         "the 1 kW cap has pulled the clocks down to where they stay (measured: the third 17 ms region after a 400 ms "
                         "prewarm still ran 13 %% faster than the fifth)")
    ap.add_argument("--transport", default="default", choices=["default", "nccl", "peer"], help="K/V exchange transport")
    ap.add_argument("--merge-mode", type=int, default=None, choices=[0, 1], help="0 separate merge kernel, 1 fused epilogue")
    ap.add_argument("--configs", default="auto", help="auto: the BASELINE.json configurations of this GPU count; none; or a comma list")
    ap.add_argument("--nccl-ctas", default="4,16", help="CTA caps for the NCCL-transport pass at N > 1 (comma list), or none")
    ap.add_argument("--block-only", default=None, metavar="B,H,Sq,Sk,D", help="only a few launches of the block kernel at this shape")
    args = ap.parse_args()
    if args.block_only:
        run_block_only(args.block_only)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs one process per GPU: launch with "
                             f"python -m torch.distributed.run --nproc-per-node {args.gpus} bench.py --gpus {args.gpus} ...")
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    run_gpu_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
