"""The ring driver on ONE GPU: `world` virtual ranks, exchange by device-to-device copy on the exchange
stream.  Exercises the step order, the receive double buffer, causal step skipping and both merge modes."""
import numpy as np
import pytest

from oracle import oracle
from ringattention_b200 import synthetic
from tests.gpu_util import assert_parity, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["auto", "256", "128"])
def rows_per_cta(request, monkeypatch):
    """Every test runs with the launcher's own choice of Q rows per CTA and with each form forced."""
    if request.param == "auto":
        monkeypatch.delenv("RING_ROWS_PER_CTA", raising=False)
    else:
        monkeypatch.setenv("RING_ROWS_PER_CTA", request.param)


def _ring_local(ra, q, k, v, world, scale, causal, merge_mode, poison=True, recv_buffers=None):
    import torch
    B, H, S, D = q.shape
    Sl = S // world
    sh = lambda x: [to_dev(x[:, :, r * Sl:(r + 1) * Sl]) for r in range(world)]
    qs, ks, vs = sh(q), sh(k), sh(v)
    ctx = ra.RingContext.create_local(world)
    ctx.set_option(ra.RING_OPT_MERGE_MODE, merge_mode)
    ctx.set_option(ra.RING_OPT_RECORD_TIMINGS, 1)
    if recv_buffers is not None:
        ctx.set_option(ra.RING_OPT_RECV_BUFFERS, recv_buffers)
        assert ctx.get_option(ra.RING_OPT_RECV_BUFFERS) == recv_buffers
    ctx.set_local_shards(ks, vs)
    outs, lses = [], []
    for r in range(world):
        out = torch.full((B, H, Sl, D), float("nan") if poison else 0.0, device="cuda")
        lse = torch.full((B, H, Sl), float("nan") if poison else 0.0, device="cuda")
        ctx.forward(qs[r], ks[r], vs[r], out, lse, causal=causal, softmax_scale=scale, rank=r)
        outs.append(out); lses.append(lse)
    ctx.synchronize()
    t = ctx.timings()
    assert len(t[0]) == world and all(x >= 0 for x in t[0])
    wait_ms, copy_ms = ctx.exchange_timings()   # the exchange of every step, split into its wait and its copy
    assert len(wait_ms) == world and all(x >= 0 for x in wait_ms) and all(x >= 0 for x in copy_ms)
    assert copy_ms[world - 1] == 0 and (world == 1 or sum(copy_ms) > 0 or causal)
    ctx.destroy()
    return torch.cat(outs, 2).cpu().numpy(), torch.cat(lses, 2).cpu().numpy()


@pytest.fixture(scope="module")
def ra():
    import ringattention_b200 as ra
    ra.device_status_reset()
    return ra


@pytest.mark.parametrize("merge_mode", [0, 1], ids=["merge-kernel", "fused-epilogue"])
@pytest.mark.parametrize("world,causal", [(1, False), (2, False), (4, False), (2, True), (4, True), (8, True)])
def test_virtual_ring_matches_oracle(ra, world, causal, merge_mode):
    B, H, D = 1, 2, 128
    S = 256 * world if world > 1 else 512
    q, k, v = synthetic.make_qkv(1000 + world, B, H, D, 0, S)
    scale = D ** -0.5
    o, lse = _ring_local(ra, q, k, v, world, scale, causal, merge_mode)
    want_o, want_lse = oracle.attention_fwd(q, k, v, scale, causal)
    assert_parity(o, lse, want_o, want_lse, f"ring world={world} causal={causal}")
    # and the blocked restatement of the reference's device algorithm agrees as well
    ring_o, ring_lse = oracle.ring_attention_fwd(q, k, v, world, scale, causal, block_n=128, round_p=True)
    assert_parity(o, lse, ring_o, ring_lse, "ring vs blocked oracle")


@pytest.mark.parametrize("recv_buffers", [0, 3], ids=["one-per-shard", "three"])
@pytest.mark.parametrize("world,causal", [(4, False), (8, True), (5, False)])
def test_virtual_ring_more_receive_buffers(ra, world, causal, recv_buffers):
    """RING_OPT_RECV_BUFFERS: one receive buffer per remote shard (no exchange waits for a compute step) or three."""
    B, H, D = 1, 2, 128
    S = 256 * world
    q, k, v = synthetic.make_qkv(1100 + world, B, H, D, 0, S)
    scale = D ** -0.5
    o, lse = _ring_local(ra, q, k, v, world, scale, causal, 1, recv_buffers=recv_buffers)
    want_o, want_lse = oracle.attention_fwd(q, k, v, scale, causal)
    assert_parity(o, lse, want_o, want_lse, f"ring world={world} recv_buffers={recv_buffers}")


def test_virtual_ring_d64_three_ranks(ra):
    B, H, D, world = 2, 2, 64, 3
    S = 384 * world
    q, k, v = synthetic.make_qkv(4242, B, H, D, 0, S)
    o, lse = _ring_local(ra, q, k, v, world, 0.125, False, 1)
    want_o, want_lse = oracle.attention_fwd(q, k, v, 0.125)
    assert_parity(o, lse, want_o, want_lse, "ring d64 world=3")


def test_virtual_ring_ragged_shard_length(ra):
    """Shards of 200 rows (not a multiple of the tile): causal ring over 3 virtual ranks."""
    B, H, D, world = 1, 2, 128, 3
    S = 200 * world
    q, k, v = synthetic.make_qkv(5151, B, H, D, 0, S)
    for causal in (False, True):
        o, lse = _ring_local(ra, q, k, v, world, D ** -0.5, causal, 1)
        want_o, want_lse = oracle.attention_fwd(q, k, v, D ** -0.5, causal)
        assert_parity(o, lse, want_o, want_lse, f"ragged ring causal={causal}")


@pytest.mark.parametrize("causal", [False, True])
def test_virtual_ring_uneven_shards(ra, causal):
    """Per-rank sequence lengths that differ (the reference's seqlen[] table, csrc/ring.h:9, :463,531)."""
    import torch
    B, H, D = 1, 2, 128
    lens = [384, 130, 512, 257]
    S, world = sum(lens), len(lens)
    q, k, v = synthetic.make_qkv(7373, B, H, D, 0, S)
    starts = np.concatenate([[0], np.cumsum(lens)])
    sh = lambda x: [to_dev(x[:, :, starts[r]:starts[r + 1]]) for r in range(world)]
    qs, ks, vs = sh(q), sh(k), sh(v)
    ctx = ra.RingContext.create_local(world)
    ctx.set_local_shards(ks, vs)
    outs, lses = [], []
    for r in range(world):
        out = torch.full((B, H, lens[r], D), float("nan"), device="cuda")
        lse = torch.full((B, H, lens[r]), float("nan"), device="cuda")
        ctx.forward(qs[r], ks[r], vs[r], out, lse, causal=causal, rank=r, seqlens=lens)
        outs.append(out); lses.append(lse)
    ctx.synchronize()
    ctx.destroy()
    want_o, want_lse = oracle.attention_fwd(q, k, v, D ** -0.5, causal)
    assert_parity(torch.cat(outs, 2).cpu().numpy(), torch.cat(lses, 2).cpu().numpy(), want_o, want_lse, "uneven shards")


@pytest.mark.parametrize("world", [1, 2, 4])
def test_virtual_ring_zigzag_causal(ra, world):
    """Zig-zag causal sharding: rank r holds chunks r and 2P-1-r; the result, put back in sequence order, is
    plain causal attention."""
    import torch
    B, H, D = 1, 2, 128
    S = 512 * world
    q, k, v = synthetic.make_qkv(8800 + world, B, H, D, 0, S)
    rows = [synthetic.zigzag_rows(r, world, S) for r in range(world)]
    sh = lambda x: [to_dev(x[:, :, rows[r]]) for r in range(world)]
    qs, ks, vs = sh(q), sh(k), sh(v)
    ctx = ra.RingContext.create_local(world)
    ctx.set_option(ra.RING_OPT_CAUSAL_ZIGZAG, 1)
    ctx.set_local_shards(ks, vs)
    got_o = np.empty((B, H, S, D), np.float32); got_l = np.empty((B, H, S), np.float32)
    outs = []
    for r in range(world):
        out = torch.full((B, H, S // world, D), float("nan"), device="cuda")
        lse = torch.full((B, H, S // world), float("nan"), device="cuda")
        ctx.forward(qs[r], ks[r], vs[r], out, lse, causal=True, rank=r)
        outs.append((out, lse))
    ctx.synchronize()
    for r in range(world):
        got_o[:, :, rows[r]] = outs[r][0].cpu().numpy(); got_l[:, :, rows[r]] = outs[r][1].cpu().numpy()
    ctx.destroy()
    want_o, want_lse = oracle.attention_fwd(q, k, v, D ** -0.5, True)
    assert_parity(got_o, got_l, want_o, want_lse, f"zig-zag world={world}")


def test_context_rejects_mismatched_calls(ra):
    import torch
    ctx = ra.RingContext.create_local(2)
    x = torch.zeros((1, 1, 128, 64), dtype=torch.float16, device="cuda")
    out = torch.zeros((1, 1, 128, 64), device="cuda")
    with pytest.raises(ra.RingError) as e:          # shards never registered
        ctx.forward(x, x, x, out, rank=0)
    assert e.value.code == -1
    p = ra.set_params_fprop(x, x, x, out, 3, 0, [128, 128, 128], 64)
    with pytest.raises(ra.RingError):               # npes differs from the context's world
        ctx.forward_params(p)
    p = ra.set_params_fprop(x, x, x, out, 2, 0, [128, 0], 64)
    with pytest.raises(ra.RingError):               # a rank without rows
        ctx.forward_params(p)
    ctx.destroy()


@pytest.mark.parametrize("chunks", [1, 3, 8])
def test_host_buffer_forward_matches_oracle(ra, chunks):
    """ring_attention_fwd_host: pinned host tensors in and out, slabs pipelined in chunks."""
    import torch
    B, H, S, D = 2, 4, 256, 128
    q, k, v = synthetic.make_qkv(808, B, H, D, 0, S)
    hq, hk, hv = (torch.from_numpy(x).pin_memory() for x in (q, k, v))
    ho = torch.full((B, H, S, D), float("nan")).pin_memory()
    hl = torch.full((B, H, S), float("nan")).pin_memory()
    ctx = ra.RingContext.create(0, 1, None)
    for _ in range(2):  # the second call reuses the staging buffers
        ho.fill_(float("nan")); hl.fill_(float("nan"))
        ctx.forward_host(hq, hk, hv, ho, hl, chunks=chunks, causal=True)
        ctx.synchronize()
        want_o, want_lse = oracle.attention_fwd(q, k, v, D ** -0.5, True)
        assert_parity(ho.numpy(), hl.numpy(), want_o, want_lse, f"host forward chunks={chunks}")
    ctx.destroy()


def test_reference_driver_executable(ra):
    """The C++ driver that mirrors the reference's main() (csrc/ring_attention.cu:750-790): its 8x8 corner must be
    the attention of the deterministic fill (:731-741), and it reports a time per call."""
    import os
    import re
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ringattention_b200", "ring_attention_main")
    env = dict(os.environ, RING_SEQ="1024", RING_WARMUP="2", RING_LOOPS="3")
    res = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = res.stdout.strip().splitlines()
    assert lines[0] == "mype: 0 success" and lines[-1].startswith("elapsedtime=")
    corner = np.array([[float(x) for x in ln.split()] for ln in lines[1:9]], dtype=np.float32)
    f = oracle.fill_with_num(1024, 64)[None, None]
    want, _ = oracle.attention_fwd(f, f, f, 64 ** -0.5)
    assert np.abs(corner - want[0, 0, :8, :8]).max() <= 2e-3 * max(1.0, float(np.abs(want).max()))
    assert float(re.sub("elapsedtime=", "", lines[-1])) > 0
