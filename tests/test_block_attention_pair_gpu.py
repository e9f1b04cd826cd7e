"""The CTA-pair forms of the block kernel (RING_PAIR=1 / 2: clusters of two CTAs, tcgen05 cta_group::2, head dimension
128, one or two softmax threads per Q row) against the CPU oracle, through the same C-ABI entry points as the one-CTA form."""
import numpy as np
import pytest

from oracle import oracle
from ringattention_b200 import synthetic
from tests.gpu_util import assert_parity, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["1", "2"], ids=["one-thread-per-row", "two-threads-per-row"])
def pair_form(request, monkeypatch):
    monkeypatch.setenv("RING_PAIR", request.param)


def _block(q, k, v, scale, **kw):
    import torch
    import ringattention_b200 as ra
    B, H, Sq, D = q.shape
    o = torch.full((B, H, Sq, D), float("nan"), device="cuda")
    lse = torch.full((B, H, Sq), float("nan"), device="cuda")
    ra.device_status_reset()
    ra.attention_block_fwd(to_dev(q), to_dev(k), to_dev(v), o, lse, softmax_scale=scale, **kw)
    assert ra.device_status() == 0
    return o.cpu().numpy(), lse.cpu().numpy()


@pytest.mark.parametrize("shape", [(1, 1, 128, 128), (1, 2, 256, 256), (2, 3, 256, 384), (1, 1, 384, 1280), (1, 2, 512, 128),
                                   (1, 1, 200, 333), (1, 3, 300, 1000), (1, 1, 257, 64), (1, 1, 1, 1), (1, 1, 129, 127)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_pair_form_matches_oracle(shape, causal):
    """Whole and ragged lengths, one CTA of a pair without rows (Sq <= 128 modulo 256), more blocks than ring slots."""
    B, H, Sq, Sk = shape
    D = 128
    q = synthetic.make_shard("q", 31, B, H, D, 0, Sq)
    k = synthetic.make_shard("k", 31, B, H, D, 0, Sk)
    v = synthetic.make_shard("v", 31, B, H, D, 0, Sk)
    scale = D ** -0.5
    q_off = max(Sk - Sq, 0) if causal else 0
    o, lse = _block(q, k, v, scale, causal=causal, q_off=q_off)
    want_o, want_l = oracle.attention_fwd(q, k, v, scale, causal=causal, q_off=q_off)
    assert_parity(o, lse, want_o, want_l, f"pair form {shape} causal={causal}")


@pytest.mark.parametrize("offs", [(0, 0), (256, 0), (0, 256), (128, 384), (1024, 0), (0, 1024)], ids=lambda o: f"q{o[0]}k{o[1]}")
def test_pair_form_causal_offsets(offs):
    """Shards anywhere relative to the diagonal: fully visible, fully masked (O = 0, LSE = -inf) and straddling."""
    B, H, Sq, Sk, D = 1, 2, 384, 512, 128
    q = synthetic.make_shard("q", 32, B, H, D, offs[0], Sq)
    k = synthetic.make_shard("k", 32, B, H, D, offs[1], Sk)
    v = synthetic.make_shard("v", 32, B, H, D, offs[1], Sk)
    o, lse = _block(q, k, v, D ** -0.5, causal=True, q_off=offs[0], k_off=offs[1])
    want_o, want_l = oracle.attention_fwd(q, k, v, D ** -0.5, causal=True, q_off=offs[0], k_off=offs[1])
    assert_parity(o, lse, want_o, want_l, f"pair form offsets {offs}")
    dead = np.isneginf(want_l)
    assert np.all(o[dead] == 0)


@pytest.mark.parametrize("gain", [0.5, 3.0])
def test_pair_form_rescale_paths_and_merge(gain):
    """Large scores drive the lazy rescale of O (the maximum is handed between the two warpgroups of a row); then a
    second K/V shard is folded into the first result by the kernel's own epilogue."""
    import torch
    import ringattention_b200 as ra
    B, H, Sq, Sk, D = 1, 2, 256, 1024, 128
    scale = D ** -0.5
    q = synthetic.make_shard("q", 33, B, H, D, 0, Sq, gain)
    k = synthetic.make_shard("k", 33, B, H, D, 0, 2 * Sk, gain)
    v = synthetic.make_shard("v", 33, B, H, D, 0, 2 * Sk)
    o = torch.full((B, H, Sq, D), float("nan"), device="cuda")
    lse = torch.full((B, H, Sq), float("nan"), device="cuda")
    ra.device_status_reset()
    tq = to_dev(q)
    ra.attention_block_fwd(tq, to_dev(k[:, :, :Sk]), to_dev(v[:, :, :Sk]), o, lse, softmax_scale=scale)
    ra.attention_block_fwd(tq, to_dev(k[:, :, Sk:]), to_dev(v[:, :, Sk:]), o, lse, softmax_scale=scale, merge=True)
    assert ra.device_status() == 0
    want_o, want_l = oracle.attention_fwd(q, k, v, scale)
    # a stale maximum leaves the dominant probability of a nearly one-hot row slightly off 1.0 in fp16: |dO| <= |v| * 5e-4
    got_o, got_l = o.cpu().numpy(), lse.cpu().numpy()
    assert np.abs(got_o - want_o).max() <= (2e-3 if gain < 1 else 4e-3)
    assert np.abs(got_l - want_l).max() <= 1e-4


def test_pair_form_ring_and_bits(monkeypatch):
    """The ring driver over the pair form (three virtual ranks, causal), and run-to-run bit equality."""
    import torch
    import ringattention_b200 as ra
    B, H, D, world, Sl = 1, 2, 128, 3, 256
    S = Sl * world
    scale = D ** -0.5
    q, k, v = synthetic.make_qkv(34, B, H, D, 0, S)

    def ring():
        sh = lambda x: [to_dev(x[:, :, r * Sl:(r + 1) * Sl]) for r in range(world)]
        qs, ks, vs = sh(q), sh(k), sh(v)
        ctx = ra.RingContext.create_local(world)
        ctx.set_local_shards(ks, vs)
        outs, lses = [], []
        for r in range(world):
            out = torch.full((B, H, Sl, D), float("nan"), device="cuda")
            lse = torch.full((B, H, Sl), float("nan"), device="cuda")
            ctx.forward(qs[r], ks[r], vs[r], out, lse, causal=True, softmax_scale=scale, rank=r)
            outs.append(out); lses.append(lse)
        ctx.synchronize()
        ctx.destroy()
        return torch.cat(outs, 2).cpu().numpy(), torch.cat(lses, 2).cpu().numpy()

    o1, l1 = ring()
    want_o, want_l = oracle.attention_fwd(q, k, v, scale, causal=True)
    assert_parity(o1, l1, want_o, want_l, "pair form, virtual ring")
    o2, l2 = ring()
    assert np.array_equal(o1, o2) and np.array_equal(l1, l2)
