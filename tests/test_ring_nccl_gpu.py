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


def _run(world, config, merge_mode, tmp_path, timeout=1500, transport="default"):
    out = os.path.join(str(tmp_path), f"{config}_{merge_mode}_{transport}.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "ring_nccl_worker.py"), "--config", config, "--merge-mode", str(merge_mode), "--out", out,
           "--transport", transport]
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
