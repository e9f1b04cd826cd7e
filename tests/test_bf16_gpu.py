"""bf16 inputs (csrc/kernel_traits.h:27-30 of the reference anticipates them) against the CPU oracle's bf16 path:
the same fp64 attention after an exact widening of the bf16 bit patterns.

Tolerance.  The kernel rounds the probabilities P to the input format before P V (as the reference does,
csrc/ring_attention.cu:604); with bf16 that is 8 significant bits, a relative error of at most 2^-9 per
element, while the row sum uses the unrounded values.  Hence |dO| <= 2^-9 * max|v| for every row (reached only
when all rounding errors align) and rel-L2(O) <= 2^-9; the LSE does not see P's rounding and keeps the 1e-4 bar.
"""
import numpy as np
import pytest

from oracle import oracle
from ringattention_b200 import synthetic

pytestmark = pytest.mark.gpu

P_ROUNDING = 2.0 ** -9
TOL_LSE = 1e-4


@pytest.fixture(autouse=True, params=["auto", "128"])
def rows_per_cta(request, monkeypatch):
    if request.param == "auto":
        monkeypatch.delenv("RING_ROWS_PER_CTA", raising=False)
    else:
        monkeypatch.setenv("RING_ROWS_PER_CTA", request.param)


def _bf16(x16):
    """fp16 synthetic values -> (torch bf16 CUDA tensor, uint16 bit patterns for the oracle), same rounding."""
    import torch
    bits = oracle.to_bf16_bits(x16.astype(np.float32))
    t = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()
    return t, bits


def _check(got_o, got_l, want_o, want_l, vmax, what):
    assert not np.isnan(got_o).any() and not np.isnan(got_l).any(), what
    fin = np.isfinite(want_l)
    assert np.array_equal(np.isneginf(got_l), np.isneginf(want_l)), what
    assert np.abs(got_o - want_o).max() <= P_ROUNDING * vmax, f"{what}: max|dO| {np.abs(got_o - want_o).max():.3e}"
    assert np.linalg.norm(got_o - want_o) / np.linalg.norm(want_o) <= P_ROUNDING, what
    assert np.abs(got_l[fin] - want_l[fin]).max() <= TOL_LSE, f"{what}: max|dLSE| {np.abs(got_l[fin] - want_l[fin]).max():.3e}"


@pytest.mark.parametrize("shape,causal,offs", [
    ((1, 2, 384, 384, 128), True, (0, 0)),       # causal diagonal
    ((2, 2, 256, 640, 64), False, (0, 0)),       # head dimension 64
    ((1, 3, 300, 1000, 128), False, (0, 0)),     # lengths that are not multiples of the tile
    ((1, 1, 129, 127, 64), True, (128, 0)),      # ragged and causal with an offset between the shards
    ((1, 2, 256, 512, 128), True, (256, 0)),     # every key visible to the later rows only
], ids=["causal", "d64", "ragged", "ragged-causal-d64", "offset"])
def test_bf16_block_vs_oracle(shape, causal, offs):
    import torch
    import ringattention_b200 as ra
    B, H, Sq, Sk, D = shape
    scale = D ** -0.5
    q = synthetic.make_shard("q", 71, B, H, D, offs[0], Sq)
    k = synthetic.make_shard("k", 71, B, H, D, offs[1], Sk)
    v = synthetic.make_shard("v", 71, B, H, D, offs[1], Sk)
    (tq, bq), (tk, bk), (tv, bv) = _bf16(q), _bf16(k), _bf16(v)
    o = torch.full((B, H, Sq, D), float("nan"), device="cuda")
    lse = torch.full((B, H, Sq), float("nan"), device="cuda")
    ra.device_status_reset()
    ra.attention_block_fwd(tq, tk, tv, o, lse, softmax_scale=scale, causal=causal, q_off=offs[0], k_off=offs[1])
    assert ra.device_status() == 0
    want_o, want_l = oracle.attention_fwd(bq, bk, bv, scale, causal=causal, q_off=offs[0], k_off=offs[1])
    vmax = float(np.abs(oracle.bf16_bits_to_f32(bv)).max())
    _check(o.cpu().numpy(), lse.cpu().numpy(), want_o, want_l, vmax, f"bf16 block {shape} causal={causal}")


@pytest.mark.parametrize("merge_mode", [0, 1], ids=["merge-kernel", "fused-epilogue"])
def test_bf16_virtual_ring_causal(merge_mode):
    """Three virtual ranks on one GPU, causal, bf16: the exchange, both merge forms and the block kernel's bf16 path."""
    import torch
    import ringattention_b200 as ra
    B, H, D, world = 1, 2, 128, 3
    Sl = 256
    S = Sl * world
    scale = D ** -0.5
    q, k, v = synthetic.make_qkv(72, B, H, D, 0, S)
    (tq, bq), (tk, bk), (tv, bv) = _bf16(q), _bf16(k), _bf16(v)
    sh = lambda t: [t[:, :, r * Sl:(r + 1) * Sl].contiguous() for r in range(world)]
    qs, ks, vs = sh(tq), sh(tk), sh(tv)
    ctx = ra.RingContext.create_local(world)
    ctx.set_option(ra.RING_OPT_MERGE_MODE, merge_mode)
    ctx.set_local_shards(ks, vs)
    outs, lses = [], []
    for r in range(world):
        out = torch.full((B, H, Sl, D), float("nan"), device="cuda")
        lse = torch.full((B, H, Sl), float("nan"), device="cuda")
        ctx.forward(qs[r], ks[r], vs[r], out, lse, causal=True, softmax_scale=scale, rank=r)
        outs.append(out); lses.append(lse)
    ctx.synchronize()
    ctx.destroy()
    want_o, want_l = oracle.attention_fwd(bq, bk, bv, scale, causal=True)
    vmax = float(np.abs(oracle.bf16_bits_to_f32(bv)).max())
    _check(torch.cat(outs, 2).cpu().numpy(), torch.cat(lses, 2).cpu().numpy(), want_o, want_l, vmax, "bf16 virtual ring")
