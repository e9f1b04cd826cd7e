"""ctypes loader for the CPU oracle (test infrastructure only).

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import
this module.  The product package never does.

The C functions restate csrc/self_attention.py:22-26 (plain attention) and
csrc/ring_attention.cu:172-245,621-633 (blocked online softmax) of the
reference; see attention_oracle.c for the line-by-line citations.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file."""
    src = os.path.join(_HERE, "attention_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        u16p = ctypes.POINTER(ctypes.c_uint16)
        f32p = ctypes.POINTER(ctypes.c_float)
        i64p = ctypes.POINTER(ctypes.c_int64)
        i64, i32, f64 = ctypes.c_int64, ctypes.c_int, ctypes.c_double
        L.oracle_attention_fwd.argtypes = [u16p, u16p, u16p, i32, i32, i64, i64, i32, f64, i32, i64, i64, i32, f32p, f32p]
        L.oracle_attention_fwd.restype = i32
        L.oracle_attention_rows.argtypes = [u16p, u16p, u16p, i32, i32, i64, i64, i32, f64, i32, i64, i64, i64p, i64, f32p, f32p]
        L.oracle_attention_rows.restype = i32
        L.oracle_lse_merge.argtypes = [f32p, f32p, f32p, f32p, i64, i32]
        L.oracle_lse_merge.restype = i32
        L.oracle_ring_attention_fwd.argtypes = [u16p, u16p, u16p, i32, i32, i64, i32, i32, i32, f64, i32, i32, f32p, f32p]
        L.oracle_ring_attention_fwd.restype = i32
        L.oracle_fill_with_num.argtypes = [u16p, i64, i64]
        L.oracle_fill_with_num.restype = i32
        L.oracle_set_input_bf16.argtypes = [i32]
        L.oracle_set_input_bf16.restype = i32
        L.oracle_set_num_threads.argtypes = [i32]
        L.oracle_set_num_threads.restype = i32
        L.oracle_num_threads.argtypes = []
        L.oracle_num_threads.restype = i32
        _lib = L
    return _lib


def _u16(a: np.ndarray):
    """fp16 arrays, or uint16 arrays holding bf16 bit patterns (numpy has no bf16 type)."""
    assert a.dtype in (np.float16, np.uint16) and a.flags["C_CONTIGUOUS"]
    lib().oracle_set_input_bf16(1 if a.dtype == np.uint16 else 0)
    return a.view(np.uint16).ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to bf16 (nearest even) and return the bit patterns as uint16: the form in which
    the functions of this module take bf16 inputs (q, k and v must then all be uint16)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def _f32(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def attention_fwd(q, k, v, scale, causal=False, q_off=0, k_off=0, accum="f64"):
    """Full attention of a Q shard against a K/V shard.  q:[B,H,Sq,D] k,v:[B,H,Sk,D] fp16.

    Returns (o [B,H,Sq,D] fp32, lse [B,H,Sq] fp32)."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    assert k.shape == (B, H, Sk, D) and v.shape == (B, H, Sk, D)
    o = np.empty((B, H, Sq, D), np.float32)
    lse = np.empty((B, H, Sq), np.float32)
    rc = lib().oracle_attention_fwd(_u16(q), _u16(k), _u16(v), B, H, Sq, Sk, D, float(scale), int(bool(causal)),
                                    int(q_off), int(k_off), 1 if accum == "f64" else 0, _f32(o), _f32(lse))
    if rc != 0:
        raise RuntimeError(f"oracle_attention_fwd failed: {rc}")
    return o, lse


def attention_rows(q, k, v, rows, scale, causal=False, q_off=0, k_off=0):
    """fp64 attention for sampled (b, h, i) rows against the full K/V.  rows: [n,3] int64."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    n = rows.shape[0]
    o = np.empty((n, D), np.float32)
    lse = np.empty((n,), np.float32)
    rc = lib().oracle_attention_rows(_u16(q), _u16(k), _u16(v), B, H, Sq, Sk, D, float(scale), int(bool(causal)),
                                     int(q_off), int(k_off), rows.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                                     n, _f32(o), _f32(lse))
    if rc != 0:
        raise RuntimeError(f"oracle_attention_rows failed: {rc}")
    return o, lse


def lse_merge(o_a, lse_a, o_b, lse_b):
    """Merge two partial (O, LSE) pairs of the same rows; returns new arrays."""
    D = o_a.shape[-1]
    o = np.ascontiguousarray(o_a, dtype=np.float32).copy()
    l = np.ascontiguousarray(lse_a, dtype=np.float32).copy()
    ob = np.ascontiguousarray(o_b, dtype=np.float32)
    lb = np.ascontiguousarray(lse_b, dtype=np.float32)
    rc = lib().oracle_lse_merge(_f32(o), _f32(l), _f32(ob), _f32(lb), l.size, D)
    if rc != 0:
        raise RuntimeError(f"oracle_lse_merge failed: {rc}")
    return o, l


def ring_attention_fwd(q, k, v, world, scale, causal=False, block_n=128, round_p=False):
    """Blocked ring attention over `world` contiguous shards of the full [B,H,S,D] tensors."""
    B, H, S, D = q.shape
    o = np.empty((B, H, S, D), np.float32)
    lse = np.empty((B, H, S), np.float32)
    rc = lib().oracle_ring_attention_fwd(_u16(q), _u16(k), _u16(v), B, H, S, D, int(world), int(block_n),
                                         float(scale), int(bool(causal)), int(bool(round_p)), _f32(o), _f32(lse))
    if rc != 0:
        raise RuntimeError(f"oracle_ring_attention_fwd failed: {rc}")
    return o, lse


def fill_with_num(m, n):
    """The reference driver's deterministic fill (csrc/ring_attention.cu:731-741) as fp16 [m,n]."""
    a = np.empty((m, n), np.float16)
    rc = lib().oracle_fill_with_num(_u16(a), m, n)
    if rc != 0:
        raise RuntimeError("oracle_fill_with_num failed")
    return a


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> int:
    """Ask OpenMP for n threads whatever OMP_NUM_THREADS says (torchrun exports 1); returns the count in use."""
    return int(lib().oracle_set_num_threads(int(n)))


def attention_numpy(q, k, v, scale, causal=False, q_off=0, k_off=0):
    """Pure numpy fp64 statement of csrc/self_attention.py:22-26 for small cases,
    independent of the C code (used to cross-check it)."""
    qf, kf, vf = (x.astype(np.float64) for x in (q, k, v))
    s = np.einsum("bhid,bhjd->bhij", qf, kf) * scale
    if causal:
        qi = q_off + np.arange(q.shape[2])[:, None]
        kj = k_off + np.arange(k.shape[2])[None, :]
        s = np.where(kj <= qi, s, -np.inf)
    with np.errstate(invalid="ignore", divide="ignore"):
        mx = s.max(axis=-1, keepdims=True)
        mx0 = np.where(np.isfinite(mx), mx, 0.0)
        p = np.exp(s - mx0)
        l = p.sum(axis=-1, keepdims=True)
        o = np.einsum("bhij,bhjd->bhid", p, vf) / np.where(l == 0, 1.0, l)
        lse = (mx0 + np.log(l))[..., 0]
    lse = np.where(l[..., 0] == 0, -np.inf, lse)
    return o.astype(np.float32), lse.astype(np.float32)
