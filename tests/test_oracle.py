"""CPU oracle checks: golden fixtures made from the reference's own statements, an
independent numpy statement, and the algebra the ring path relies on."""
import glob
import os

import numpy as np
import pytest

from oracle import oracle
from ringattention_b200 import synthetic

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _b(x):
    return np.ascontiguousarray(x[None, None])


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_golden(path):
    g = np.load(path)
    q, k, v = _b(g["q"]), _b(g["k"]), _b(g["v"])
    for accum, tol_o, tol_l in (("f64", 2e-6, 2e-6), ("f32", 2e-5, 2e-5)):
        o, lse = oracle.attention_fwd(q, k, v, float(g["scale"]), accum=accum)
        assert np.abs(o[0, 0] - g["o_f64"]).max() <= tol_o
        assert np.abs(lse[0, 0] - g["lse_f64"]).max() <= tol_l
    # the reference's own fp16 arithmetic agrees to fp16 resolution
    assert np.abs(o[0, 0] - g["o_f16"].astype(np.float32)).max() <= 4e-3


def test_golden_inputs_come_from_the_seeded_generator():
    for path in GOLDEN:
        g = np.load(path)
        S, D = g["q"].shape
        q, k, v = synthetic.make_qkv(int(g["seed"]), 1, 1, D, 0, S, float(g["gain"]))
        assert np.array_equal(q[0, 0], g["q"]) and np.array_equal(k[0, 0], g["k"]) and np.array_equal(v[0, 0], g["v"])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 2, 96, 160, 64), (2, 1, 130, 70, 128), (1, 1, 1, 1, 64)])
def test_oracle_vs_numpy(shape, causal):
    B, H, Sq, Sk, D = shape
    q = synthetic.make_shard("q", 3, B, H, D, 0, Sq)
    k = synthetic.make_shard("k", 3, B, H, D, 0, Sk)
    v = synthetic.make_shard("v", 3, B, H, D, 0, Sk)
    scale = D ** -0.5
    for q_off, k_off in ((0, 0), (40, 0), (0, 40)):
        o, lse = oracle.attention_fwd(q, k, v, scale, causal, q_off, k_off)
        o2, lse2 = oracle.attention_numpy(q, k, v, scale, causal, q_off, k_off)
        assert np.allclose(o, o2, atol=2e-6)
        assert np.array_equal(np.isneginf(lse), np.isneginf(lse2))
        fin = np.isfinite(lse2)
        assert np.allclose(lse[fin], lse2[fin], atol=2e-6)
        assert np.all(o[~fin] == 0)


def test_sampled_rows_match_full():
    B, H, S, D = 2, 3, 200, 64
    q, k, v = synthetic.make_qkv(5, B, H, D, 0, S)
    rows = synthetic.sample_rows(9, B, H, S, 40, always=(0, S - 1))
    for causal in (False, True):
        o, lse = oracle.attention_fwd(q, k, v, 0.125, causal)
        orow, lrow = oracle.attention_rows(q, k, v, rows, 0.125, causal)
        for n, (b, h, i) in enumerate(rows):
            assert np.array_equal(orow[n], o[b, h, i]) and lrow[n] == lse[b, h, i]


@pytest.mark.parametrize("world,causal", [(1, False), (2, False), (4, False), (4, True), (8, True)])
def test_blocked_ring_equals_plain_attention(world, causal):
    B, H, S, D = 1, 2, 512, 64
    q, k, v = synthetic.make_qkv(7, B, H, D, 0, S)
    scale = D ** -0.5
    o, lse = oracle.attention_fwd(q, k, v, scale, causal)
    o2, lse2 = oracle.ring_attention_fwd(q, k, v, world, scale, causal, block_n=64)
    assert np.abs(o - o2).max() <= 5e-6
    assert np.abs(lse - lse2).max() <= 5e-6
    # rounding P to fp16 before PV (what the device code does) stays inside the parity budget
    o3, lse3 = oracle.ring_attention_fwd(q, k, v, world, scale, causal, block_n=128, round_p=True)
    assert np.abs(o - o3).max() <= 2e-3
    assert np.linalg.norm(o - o3) / np.linalg.norm(o) <= 1e-3
    assert np.abs(lse - lse3).max() <= 1e-5


def test_merge_of_halves_equals_whole():
    B, H, S, D = 1, 2, 256, 128
    q, k, v = synthetic.make_qkv(21, B, H, D, 0, S)
    scale = D ** -0.5
    o, lse = oracle.attention_fwd(q, k, v, scale)
    h = S // 2
    oa, la = oracle.attention_fwd(q, k[:, :, :h].copy(), v[:, :, :h].copy(), scale)
    ob, lb = oracle.attention_fwd(q, k[:, :, h:].copy(), v[:, :, h:].copy(), scale)
    om, lm = oracle.lse_merge(oa, la, ob, lb)
    assert np.abs(om - o).max() <= 2e-6 and np.abs(lm - lse).max() <= 2e-6
    # merge is commutative, and a fully masked partial (-inf) is the identity
    om2, lm2 = oracle.lse_merge(ob, lb, oa, la)
    assert np.allclose(om, om2, atol=1e-6) and np.allclose(lm, lm2, atol=1e-6)
    empty_o = np.zeros_like(oa)
    empty_l = np.full_like(la, -np.inf)
    o3, l3 = oracle.lse_merge(oa, la, empty_o, empty_l)
    assert np.array_equal(o3, oa) and np.array_equal(l3, la)
    o4, l4 = oracle.lse_merge(empty_o, empty_l, empty_o, empty_l)
    assert np.all(o4 == 0) and np.all(np.isneginf(l4))


def test_causal_merge_across_shards():
    """Contiguous causal sharding: merging the per-source partials reproduces global causal."""
    B, H, S, D, P = 1, 1, 384, 64, 3
    q, k, v = synthetic.make_qkv(33, B, H, D, 0, S)
    scale = 0.125
    o, lse = oracle.attention_fwd(q, k, v, scale, True)
    Sl = S // P
    for r in range(P):
        qs = q[:, :, r * Sl:(r + 1) * Sl].copy()
        acc = None
        for step in range(P):
            src = (r + step) % P
            ks, vs = (x[:, :, src * Sl:(src + 1) * Sl].copy() for x in (k, v))
            part = oracle.attention_fwd(qs, ks, vs, scale, True, r * Sl, src * Sl)
            acc = part if acc is None else oracle.lse_merge(acc[0], acc[1], part[0], part[1])
        assert np.abs(acc[0] - o[:, :, r * Sl:(r + 1) * Sl]).max() <= 2e-6
        assert np.abs(acc[1] - lse[:, :, r * Sl:(r + 1) * Sl]).max() <= 2e-6


def test_fill_with_num_matches_formula():
    a = oracle.fill_with_num(70, 64)
    i, j = np.meshgrid(np.arange(70), np.arange(64), indexing="ij")
    want = (i / 130.0 + j / 110.0 + i * j / 600.0).astype(np.float32).astype(np.float16)
    assert np.array_equal(a, want)


def test_bad_arguments_are_rejected():
    q = np.zeros((1, 1, 4, 64), np.float16)
    with pytest.raises(RuntimeError):
        oracle.attention_rows(q, q, q, np.array([[0, 0, 9]]), 1.0)
    with pytest.raises(RuntimeError):
        oracle.ring_attention_fwd(q, q, q, 3, 1.0)
