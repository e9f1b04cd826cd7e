"""Seeded synthetic Q/K/V for the ring-attention forward.

The generator is counter based: the values of rows [r0, r0 + n) of tensor `which`
for head (b, h) depend only on (seed, which, b, h, global row block), never on how
the sequence is sharded.  Every rank, the CPU oracle and the tests can therefore
regenerate any slice of the same global tensors independently.

Values are i.i.d. N(0, 1) * gain drawn in fp32 and rounded to fp16 (round to nearest
even); layout is [B, H, rows, D], the per-(b,h) slab being the [seqlen, dim] row-major
matrix the reference's kernel takes (csrc/ring_attention.cu:422-426).
"""
from __future__ import annotations

import numpy as np

ROW_BLOCK = 1024  # rows per independently keyed random stream
TENSOR_IDS = {"q": 0, "k": 1, "v": 2}


def _stream(seed: int, which: int, bh: int, block: int) -> np.random.Generator:
    key = np.array([(int(seed) << 8) | (which & 0xFF), (int(bh) << 32) | int(block)], dtype=np.uint64)
    return np.random.Generator(np.random.Philox(key=key))


def make_shard(which: str, seed: int, B: int, H: int, D: int, row_start: int, rows: int,
               gain: float = 1.0, out: np.ndarray | None = None) -> np.ndarray:
    """fp16 [B, H, rows, D] slice [row_start, row_start + rows) of global tensor `which`."""
    tid = TENSOR_IDS[which]
    if out is None:
        out = np.empty((B, H, rows, D), dtype=np.float16)
    assert out.shape == (B, H, rows, D) and out.dtype == np.float16
    first_blk = row_start // ROW_BLOCK
    last_blk = (row_start + rows - 1) // ROW_BLOCK if rows > 0 else first_blk - 1
    for b in range(B):
        for h in range(H):
            bh = b * H + h
            for blk in range(first_blk, last_blk + 1):
                vals = _stream(seed, tid, bh, blk).standard_normal((ROW_BLOCK, D), dtype=np.float32)
                if gain != 1.0:
                    vals *= np.float32(gain)
                g0 = blk * ROW_BLOCK
                lo = max(g0, row_start)
                hi = min(g0 + ROW_BLOCK, row_start + rows)
                out[b, h, lo - row_start:hi - row_start, :] = vals[lo - g0:hi - g0, :]
    return out


def make_qkv(seed: int, B: int, H: int, D: int, row_start: int, rows: int, gain: float = 1.0):
    """(q, k, v) shards for the same row range."""
    return tuple(make_shard(w, seed, B, H, D, row_start, rows, gain) for w in ("q", "k", "v"))


def sample_rows(seed: int, B: int, H: int, S: int, n: int, always=()):
    """n distinct-ish seeded (b, h, i) probes of a [B, H, S] index space, plus `always` rows
    (first/last row of a shard, rows next to the causal diagonal) for every head 0."""
    rng = np.random.Generator(np.random.Philox(key=np.array([int(seed), 0x5A17], dtype=np.uint64)))
    rows = np.stack([rng.integers(0, B, n), rng.integers(0, H, n), rng.integers(0, S, n)], axis=1)
    extra = np.array([[0, 0, int(i)] for i in always if 0 <= int(i) < S], dtype=np.int64).reshape(-1, 3)
    return np.concatenate([extra, rows.astype(np.int64)], axis=0)


def make_head(which: str, seed: int, H: int, D: int, b: int, h: int, row_start: int, rows: int,
              gain: float = 1.0) -> np.ndarray:
    """fp16 [rows, D]: rows [row_start, row_start + rows) of head (b, h) of global tensor `which`
    (identical values to the same slice of make_shard)."""
    tid = TENSOR_IDS[which]
    out = np.empty((rows, D), dtype=np.float16)
    bh = b * H + h
    first_blk = row_start // ROW_BLOCK
    last_blk = (row_start + rows - 1) // ROW_BLOCK if rows > 0 else first_blk - 1
    for blk in range(first_blk, last_blk + 1):
        vals = _stream(seed, tid, bh, blk).standard_normal((ROW_BLOCK, D), dtype=np.float32)
        if gain != 1.0:
            vals *= np.float32(gain)
        g0 = blk * ROW_BLOCK
        lo = max(g0, row_start)
        hi = min(g0 + ROW_BLOCK, row_start + rows)
        out[lo - row_start:hi - row_start, :] = vals[lo - g0:hi - g0, :]
    return out


def zigzag_rows(rank: int, world: int, S: int) -> np.ndarray:
    """Global row indices held by `rank` under zig-zag sharding: the sequence of S rows is cut into 2 * world
    chunks and the rank holds chunk `rank` followed by chunk `2 * world - 1 - rank`."""
    chunk = S // (2 * world)
    a = np.arange(rank * chunk, (rank + 1) * chunk)
    b = np.arange((2 * world - 1 - rank) * chunk, (2 * world - rank) * chunk)
    return np.concatenate([a, b])
