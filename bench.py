#!/usr/bin/env python
"""Benchmark of the ring-attention forward (the one hot path of this repository).

    python bench.py --gpus N --steps K --warmup W            # this implementation (CUDA, sm_100a)
    python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference path

For N > 1 it is launched one process per GPU (torchrun); ranks shard the sequence, exchange K/V over
NCCL and rank 0 prints ONE JSON line.  A "step" is one ring-attention forward over every rank's shard.

Workload (config.workload): configs[1] of BASELINE.json at one GPU -- batch 2, 16 heads, head_dim 128,
fp16, non-causal, 8192 sequence rows per GPU; with N GPUs the total sequence is 8192 * N (weak scaling:
rows per GPU fixed).  Inputs are seeded synthetic N(0,1) values; Q, K and V together are 192 MiB per
GPU, larger than the 126 MB L2, so no explicit L2 flush is needed between timed iterations.
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

# dram__bytes_read.sum + dram__bytes_write.sum of ONE block-kernel launch at the bench shape, from the ncu
# capture summarised in profiles/ (None until a capture exists).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 301.9e6  # 201.7 MB read + 100.2 MB written (profiles/block_attention_b2_h16_s8192_d128.md)


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
def time_cpu_port(rows_target_s: float = 12.0):
    """Times the CPU restatement of the reference path (oracle port, fp32 accumulate, OpenMP on every
    host core) on a bounded sample of the bench workload: the first R query rows of head (0, 0) against
    all 8192 keys of that head.  Returns (tflops, cores, sample description, seconds)."""
    from oracle import oracle
    from ringattention_b200 import synthetic
    q, k, v = synthetic.make_qkv(SEED, 1, 1, D, 0, S_LOCAL)
    scale = D ** -0.5
    probe = 256
    t0 = time.perf_counter()
    oracle.attention_fwd(np.ascontiguousarray(q[:, :, :probe]), k, v, scale, accum="f32")
    dt = max(time.perf_counter() - t0, 1e-4)
    rows = int(min(S_LOCAL, max(probe, probe * rows_target_s / dt)))
    rows = max(128, rows // 128 * 128)
    t0 = time.perf_counter()
    oracle.attention_fwd(np.ascontiguousarray(q[:, :, :rows]), k, v, scale, accum="f32")
    dt = time.perf_counter() - t0
    fl = 4.0 * D * rows * S_LOCAL
    return fl / dt / 1e12, oracle.num_threads(), f"first {rows} query rows of head (0,0) x all {S_LOCAL} keys, fp32 accumulate", dt


def run_reference_arm(args, rank: int):
    """--impl reference: the reference's CPU implementation of the path.  The reference itself has no CPU
    attention and its CUDA source does not compile, so this is the oracle port (kind = "port")."""
    if rank != 0:
        return
    vals, secs = [], []
    cores, sample = 1, ""
    per_step = max(2.0, min(12.0, 120.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        tf, cores, sample, dt = time_cpu_port(per_step)
        if i >= args.warmup:
            vals.append(tf); secs.append(dt)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.mean(secs)) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(1), "batch": B, "heads": H, "seq_local": S_LOCAL, "head_dim": D,
                   "causal": False, "note": "each step is a bounded sample of the workload, extrapolation-free: value = sample flops / sample time"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(world: int) -> str:
    return (f"BASELINE configs[1] shape per GPU: batch {B}, heads {H}, head_dim {D}, fp16, non-causal, "
            f"{S_LOCAL} rows/GPU, total seq {S_LOCAL * world}")


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

    # ---- inputs: this rank's rows of the global seeded tensors, in pinned host memory and on the device
    hq, hk, hv = (torch.from_numpy(x).pin_memory() for x in synthetic.make_qkv(SEED, B, H, D, rank * S_LOCAL, S_LOCAL))
    q, k, v = (x.to(dev) for x in (hq, hk, hv))
    out = torch.empty((B, H, S_LOCAL, D), dtype=torch.float32, device=dev)
    lse = torch.empty((B, H, S_LOCAL), dtype=torch.float32, device=dev)
    h_out = torch.empty(out.shape, dtype=torch.float32).pin_memory()
    h_lse = torch.empty(lse.shape, dtype=torch.float32).pin_memory()
    scale = D ** -0.5
    stream = torch.cuda.current_stream()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        ctx.forward(q, k, v, out, lse, softmax_scale=scale)

    def step_e2e():
        # the public host-buffer call: pinned Q, K, V in, pinned O, LSE out, copies inside the timed region
        ctx.forward_host(hq, hk, hv, h_out, h_lse, chunks=args.e2e_chunks, softmax_scale=scale)

    per_step = {}  # name of the timed function -> this rank's per-step milliseconds of its last timed run

    def timed(fn, steps):
        barrier()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record(stream)
        for i in range(steps):
            fn()
            marks[i + 1].record(stream)
        marks[-1].synchronize()
        barrier()
        ms = marks[0].elapsed_time(marks[-1])
        per_step[fn.__name__] = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
        if dist is not None:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step_resident()
    ctx.synchronize()
    # Power-steady state: a B200 runs a short burst at 1965 MHz and settles near 1.6 GHz under its 1 kW cap after
    # some hundred milliseconds of this kernel.  With N GPUs a step is N times longer, so without this phase the
    # N = 1 line would be a burst number and the N = 8 line a sustained one.  Untimed; same count on every rank.
    probe_ms = timed(step_resident, 3) / 3
    n_pre = int(min(2000, max(0, args.prewarm_ms / max(probe_ms, 1e-3))))
    for _ in range(n_pre):
        step_resident()
    ctx.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ra.kernel_launch_count()
    total_ms = timed(step_resident, args.steps)
    steps_ms = list(per_step["step_resident"])
    launches = ra.kernel_launch_count() - launches0
    ctx.synchronize()  # also checks the device status word
    compute_ms, comm_ms, exposed_ms = ctx.timings()  # of the last timed step
    clocks = sampler.stop() if rank == 0 else None

    # ---- dominant kernel alone (block attention, one shard against one shard), CUDA events over a batch of
    # launches, taken right after the timed region so that it sees the same power-steady clocks
    reps = 50
    for _ in range(3):
        ra.attention_block_fwd(q, k, v, out, lse, softmax_scale=scale)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        ra.attention_block_fwd(q, k, v, out, lse, softmax_scale=scale)
    e1.record(stream)
    e1.synchronize()
    k1_ms = e0.elapsed_time(e1) / reps
    assert ra.device_status() == 0

    # ---- end to end: host buffers in, host buffers out, every step
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps)
    ctx.synchronize()

    # ---- merge kernel alone (HBM bound), for the record
    o2, l2 = torch.empty_like(out), torch.empty_like(lse)
    ra.attention_block_fwd(q, k, v, o2, l2, softmax_scale=scale)
    for _ in range(3):
        ra.lse_merge(out, lse, o2, l2)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(reps):
        ra.lse_merge(out, lse, o2, l2)
    e1.record(stream)
    e1.synchronize()
    k2_ms = e0.elapsed_time(e1) / reps

    if rank == 0:
        peaks = load_peaks()
        ms_per_step = total_ms / args.steps
        job_flops = flops_per_rank(world) * world
        value = job_flops / (ms_per_step * 1e-3) / 1e12
        e2e_value = job_flops / (e2e_ms / args.steps * 1e-3) / 1e12
        k1_flops = 4.0 * D * B * H * S_LOCAL * S_LOCAL
        k1_tflops = k1_flops / (k1_ms * 1e-3) / 1e12
        k2_bytes = (3 * D + 3) * 4.0 * B * H * S_LOCAL
        cpu_tf, cores, sample, _ = time_cpu_port(12.0) if world == 1 else (None, None, None, None)
        step_ms = sum(compute_ms) + sum(exposed_ms)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "ms_per_step_median_rank0": statistics.median(steps_ms),
            "ms_per_step_min_rank0": min(steps_ms), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": workload_name(world), "batch": B, "heads": H, "seq_local": S_LOCAL, "head_dim": D,
                       "causal": False, "parallelism": f"ring{world} (sequence sharded, double-buffered K/V exchange on a side stream)",
                       "kv_transport": transport,
                       "l2": "inputs (192 MiB of Q,K,V per GPU) exceed the 126 MB L2; no flush between iterations",
                       "prewarm": f"{n_pre} untimed steps (~{args.prewarm_ms:.0f} ms) before the timed region, to reach the power-capped steady clocks",
                       "merge_mode": "separate kernel" if args.merge_mode == 0 else "fused epilogue"},
            "per_gpu_tflops": value / world,
            "roofline": {"bound": "tensor", "kernel": "ring_block_attention_kernel<128,256,128,12,half>",
                         "achieved": k1_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": k1_tflops / peaks["tflops"],
                         "peak_source": peaks["source"] + " (cuBLAS bf16 burst; kernel timed in the power-steady state)",
                         "frac_of_sustained_peak": (k1_tflops / peaks["tflops_sustained"]) if peaks["tflops_sustained"] else None,
                         "frac_of_nominal_2250": k1_tflops / 2250.0,
                         "flops_per_launch": k1_flops, "ms_per_launch": k1_ms, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH},
            "merge_kernel": {"bound": "hbm", "achieved": k2_bytes / (k2_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": k2_bytes / (k2_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "ms_per_launch": k2_ms},
            "exchange": {"compute_ms_per_ring_step": compute_ms, "comm_ms_per_ring_step": comm_ms,
                         "exposed_ms_per_ring_step": exposed_ms,
                         "exposed_frac": (sum(exposed_ms) / step_ms) if step_ms > 0 else 0.0,
                         "kv_bytes_per_ring_step": 2 * B * H * S_LOCAL * D * 2},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 3 * B * H * S_LOCAL * D * 2 * world,
                    "d2h_bytes_per_step": (B * H * S_LOCAL * D * 4 + B * H * S_LOCAL * 4) * world},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if cpu_tf is not None:
            line["cpu_baseline"] = {"value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)

    ctx.destroy()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-chunks", type=int, default=8, help="(batch, head) groups the host-buffer forward pipelines")
    ap.add_argument("--prewarm-ms", type=float, default=400.0, help="untimed work before the timed region (power-steady clocks)")
    ap.add_argument("--transport", default="default", choices=["default", "nccl", "peer"], help="K/V exchange transport")
    ap.add_argument("--merge-mode", type=int, default=None, choices=[0, 1], help="0 separate merge kernel, 1 fused epilogue")
    args = ap.parse_args()
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
