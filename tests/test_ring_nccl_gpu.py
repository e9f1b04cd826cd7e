"""Multi-GPU parity of the NCCL ring (one process per GPU through torchrun).  Needs >= 2 GPUs; the cases
that fit the visible GPU count run, the others skip.  Full-size BASELINE configurations c2 (2 GPUs),
c3 (4 GPUs), c4 and c5 (8 GPUs) are checked on seeded sample rows against the fp64 oracle."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    import torch
    return torch.cuda.device_count()


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _run(world, config, merge_mode, tmp_path, timeout=1500, transport="default", recv_buffers=2):
    out = os.path.join(str(tmp_path), f"{config}_{merge_mode}_{transport}.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "ring_nccl_worker.py"), "--config", config, "--merge-mode", str(merge_mode), "--out", out,
           "--transport", transport, "--recv-buffers", str(recv_buffers)]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    r = json.load(open(out))
    assert r["ok"], r
    return r


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("transport", ["nccl", "peer"])
@pytest.mark.parametrize("config,merge_mode", [("small", 1), ("small", 0), ("small_causal", 1)])
def test_ring_small(world, config, merge_mode, transport, tmp_path):
    """Both transports of the exchange: NCCL send/recv and copy-engine pushes into IPC-shared buffers."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, config, merge_mode, tmp_path, transport=transport)
    assert r["transport"] == transport


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("transport", ["nccl", "peer"])
@pytest.mark.parametrize("config", ["uneven", "uneven_causal", "bf16", "bf16_causal_d64"])
def test_ring_uneven_shards_and_bf16(world, config, transport, tmp_path):
    """Shards of different lengths per rank (the receive layout is sized for the longest) and bf16 inputs, on real
    ranks, for both transports."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, config, 1, tmp_path, transport=transport)
    assert r["transport"] == transport


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ring_small_zigzag(world, tmp_path):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, "small_zigzag", 1, tmp_path)


@pytest.mark.parametrize("config,world", [("c2", 2), ("c3", 4), ("c4", 8), ("c4_zigzag", 8), ("c5", 8)])
def test_nccl_ring_baseline_configs(config, world, tmp_path):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, config, 1, tmp_path)
    print(json.dumps(r))


def test_reference_driver_two_pes(tmp_path):
    """The reference's own experiment (`nvshmrun -n 2 build/ring_attention`, makefile:1-2; main,
    csrc/ring_attention.cu:750-790) with this library's driver executable: two processes, one GPU each, every PE
    holding the same deterministic fill; rank 0's 8x8 corner must be the attention of its Q over the 2 x S rows."""
    import numpy as np
    from oracle import oracle
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    exe = os.path.join(ROOT, "ringattention_b200", "ring_attention_main")
    S = 1024
    idf = os.path.join(str(tmp_path), "ring_id")
    procs = []
    for r in range(2):
        env = dict(os.environ, RING_SEQ=str(S), RING_WARMUP="2", RING_LOOPS="3", RING_WORLD="2", RING_RANK=str(r),
                   RING_ID_FILE=idf, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([exe], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        try:
            o, e = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for x in procs:
                x.kill()          # the exact processes this test started
            raise
        assert p.returncode == 0, o + e
        outs.append(o)
    keep = lambda text: [ln for ln in text.strip().splitlines() if not ln.startswith("NCCL version")]  # NCCL's own banner
    lines = keep(outs[0])
    assert lines[0] == "mype: 0 success" and lines[-1].startswith("elapsedtime=")
    assert keep(outs[1])[0] == "mype: 1 success"
    corner = np.array([[float(x) for x in ln.split()] for ln in lines[1:9]], dtype=np.float32)
    f = oracle.fill_with_num(S, 64)
    kv = np.concatenate([f, f], axis=0)[None, None]
    want, _ = oracle.attention_fwd(f[None, None], kv, kv, 64 ** -0.5)
    assert np.abs(corner - want[0, 0, :8, :8]).max() <= 2e-3 * max(1.0, float(np.abs(want).max()))


def test_peer_stops_rank_aborts_and_leaves(tmp_path):
    """Recovery after a detected failure, on two real ranks (see tests/ring_abort_worker.py): the rank whose peer sat
    out a forward sees RING_ERR_HOST_TIMEOUT, aborts, is refused further forwards and destroys its context in bounded
    time; both processes exit 0 with a clean device status."""
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "ring_abort_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    recs = [json.loads(ln) for ln in res.stdout.splitlines() if ln.startswith("{")]
    by_rank = {r["rank"]: r for r in recs}
    if any("skipped" in r for r in recs):
        pytest.skip(recs[0].get("skipped", "peer-copy transport unavailable"))
    r0 = by_rank[0]
    assert r0["timeout_code"] == -7 and "exchange" in r0["timeout_message"], r0    # RING_ERR_HOST_TIMEOUT
    assert 0.4 <= r0["waited_s"] <= 3.0
    assert r0["refused_after_abort"] is True
    assert r0["destroy_s"] <= 8.0
    assert r0["device_status"] == 0 and by_rank[1]["device_status"] == 0


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("transport", ["nccl", "peer"])
@pytest.mark.parametrize("config", ["small", "uneven_causal"])
def test_ring_one_receive_buffer_per_shard(world, config, transport, tmp_path):
    """RING_OPT_RECV_BUFFERS = 0 on real ranks: every exchange has a buffer of its own, none waits for a compute step."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, config, 1, tmp_path, transport=transport, recv_buffers=0)
    assert r["transport"] == transport
