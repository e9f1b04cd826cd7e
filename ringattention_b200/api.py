"""Python host side of the B200 ring-attention forward.

Mirrors the operator interface of the reference for this path, over the C ABI of
include/ring_attention_b200.h:
  * ring_attention(q, k, v, out, npes, mype, seqlen, dim, max_seq) -- same name, argument order
    and meaning as csrc/ring_attention.cu:706 of the reference (synchronous, single head);
  * Ring_fwd_params / set_params_fprop -- csrc/ring.h:5-19 and csrc/ring_attention.cu:361-395;
  * RingContext -- what nvshmem_init + the symmetric buffers provide there
    (csrc/ring_attention.cu:754-761, 391-393): communicator, side stream, receive buffers.
torch is used only for device memory, streams and the rendezvous; every computation goes through
the CUDA library, and a missing library is an error, never a fallback.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

from . import _lib
from ._lib import Ring_fwd_params, check

__all__ = [
    "ring_attention", "ring_attention_scaled", "set_params_fprop", "Ring_fwd_params", "RingContext",
    "attention_block_fwd", "lse_merge", "device_status", "device_status_reset", "kernel_launch_count",
    "attention_chunked_fwd_static", "static_status",
]


def _ptr(x, what: str = "tensor", dtypes=None) -> int:
    """Device address of a torch tensor (checked like the reference's CHECK_INPUT,
    include/attention_api.cuh:12-18) or a raw integer address."""
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        if not x.is_cuda:
            raise ValueError(f"{what} must be a CUDA tensor")
        if not x.is_contiguous():
            raise ValueError(f"{what} must be contiguous")
        if dtypes is not None and x.dtype not in dtypes:
            raise ValueError(f"{what} has dtype {x.dtype}, expected one of {dtypes}")
        return x.data_ptr()
    raise TypeError(f"{what}: expected a CUDA tensor or an integer device address")


def _half_types():
    import torch
    return (torch.float16, torch.bfloat16)


def _stream_handle(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _int_array(values: Sequence[int]):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])


def ring_attention(q, k, v, out, npes: int, mype: int, seqlen: Sequence[int], dim: int, max_seq: int) -> None:
    """The reference's entry point (csrc/ring_attention.cu:706): q, k, v [seqlen[mype], dim] fp16 on the
    device, out [seqlen[mype], dim] fp32, single head, non-causal, synchronous.  Softmax scale 1/sqrt(dim)."""
    lib = _lib.load()
    arr = _int_array(seqlen)
    check(lib.ring_attention(_ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _ptr(out, "out"), int(npes), int(mype),
                             arr, int(dim), int(max_seq)), "ring_attention")


def ring_attention_scaled(q, k, v, out, npes, mype, seqlen, dim, max_seq, softmax_scale: float) -> None:
    """ring_attention with an explicit natural-base scale (1.0 reproduces csrc/self_attention.py:22-26)."""
    lib = _lib.load()
    arr = _int_array(seqlen)
    check(lib.ring_attention_scaled(_ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _ptr(out, "out"), int(npes), int(mype),
                                    arr, int(dim), int(max_seq), float(softmax_scale)), "ring_attention_scaled")


def set_params_fprop(q, k, v, out, npes: int, mype: int, seqlen: Sequence[int], dim: int, max_seq: int = 0,
                     *, batch: int = 1, heads: int = 1, lse=None, causal: bool = False,
                     softmax_scale: Optional[float] = None, stream=None) -> Ring_fwd_params:
    """Fill a Ring_fwd_params like the reference's set_params_fprop (csrc/ring_attention.cu:361-395);
    keyword arguments cover the extension fields.  The returned struct keeps the seqlen table alive."""
    import torch
    p = Ring_fwd_params()
    arr = _int_array(seqlen)
    p._keep = arr  # ctypes does not own the pointee otherwise
    p.mype, p.npes = int(mype), int(npes)
    p.seqlen = None
    p.h_seqlen = ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))
    p.dim = int(dim)
    p.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(dim)
    p.q_ptr, p.k_ptr, p.v_ptr = (_ptr(x, n, _half_types() if hasattr(x, "dtype") else None)
                                 for x, n in ((q, "q"), (k, "k"), (v, "v")))
    p.out_ptr = _ptr(out, "out", (torch.float32,) if hasattr(out, "dtype") else None)
    p.k_buffer = p.v_buffer = None
    p.batch, p.heads = int(batch), int(heads)
    p.lse_ptr = _ptr(lse, "lse", (torch.float32,) if hasattr(lse, "dtype") else None) or None
    p.causal = int(bool(causal))
    p.is_bf16 = int(hasattr(q, "dtype") and q.dtype == torch.bfloat16)
    p.stream = _stream_handle(stream)
    return p


class RingContext:
    """Owns the communicator, the exchange stream, events, the receive double buffer and the workspace."""

    def __init__(self, handle: int, rank: int, world: int, local: bool):
        self._h = ctypes.c_void_p(handle)
        self.rank, self.world, self.local = rank, world, local
        self._keep = None

    # ---- construction -------------------------------------------------------------------------------
    @staticmethod
    def unique_id() -> bytes:
        buf = ctypes.create_string_buffer(_lib.RING_UNIQUE_ID_BYTES)
        check(_lib.load().ring_get_unique_id(buf), "ring_get_unique_id")
        return buf.raw

    @classmethod
    def create(cls, rank: int = 0, world: int = 1, unique_id: Optional[bytes] = None) -> "RingContext":
        h = ctypes.c_void_p()
        uid = ctypes.create_string_buffer(unique_id, _lib.RING_UNIQUE_ID_BYTES) if unique_id else None
        check(_lib.load().ring_ctx_create(ctypes.byref(h), int(rank), int(world), uid), "ring_ctx_create")
        return cls(h.value, rank, world, False)

    @classmethod
    def from_torch_distributed(cls, group=None) -> "RingContext":
        """One process per GPU: rank 0 makes the id, torch.distributed carries it to the others."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if world == 1:
            return cls.create(0, 1, None)
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls.create(rank, world, box[0])

    @classmethod
    def create_local(cls, world: int) -> "RingContext":
        """`world` virtual ranks on the current GPU; the exchange is a device-to-device copy."""
        h = ctypes.c_void_p()
        check(_lib.load().ring_ctx_create_local(ctypes.byref(h), int(world)), "ring_ctx_create_local")
        return cls(h.value, 0, world, True)

    def set_local_shards(self, k_shards, v_shards) -> None:
        n = self.world
        ks = (ctypes.c_void_p * n)(*[_ptr(x, "k shard") for x in k_shards])
        vs = (ctypes.c_void_p * n)(*[_ptr(x, "v shard") for x in v_shards])
        self._keep = (list(k_shards), list(v_shards))
        check(_lib.load().ring_ctx_set_local_shards(self._h, ks, vs), "ring_ctx_set_local_shards")

    # ---- options --------------------------------------------------------------------------------------
    def set_option(self, option: int, value: int) -> None:
        check(_lib.load().ring_ctx_set_option(self._h, int(option), int(value)), "ring_ctx_set_option")

    def get_option(self, option: int) -> int:
        v = ctypes.c_int(0)
        check(_lib.load().ring_ctx_get_option(self._h, int(option), ctypes.byref(v)), "ring_ctx_get_option")
        return v.value

    def set_default(self) -> None:
        """Make this the context the plain ring_attention() call uses."""
        check(_lib.load().ring_set_default_ctx(self._h), "ring_set_default_ctx")

    # ---- the forward ------------------------------------------------------------------------------------
    def forward_params(self, params: Ring_fwd_params) -> None:
        check(_lib.load().ring_attention_fwd(self._h, ctypes.byref(params)), "ring_attention_fwd")

    def forward(self, q, k, v, out, lse=None, *, causal: bool = False, softmax_scale: Optional[float] = None,
                stream=None, rank: Optional[int] = None, seqlens: Optional[Sequence[int]] = None) -> None:
        """q, k, v: [B, H, S_local, D] fp16/bf16 shards of this rank; out [B, H, S_local, D] fp32;
        lse [B, H, S_local] fp32 or None.  Asynchronous on `stream` (default: torch's current stream)."""
        B, H, S, D = q.shape
        if tuple(k.shape) != (B, H, S, D) or tuple(v.shape) != (B, H, S, D) or tuple(out.shape) != (B, H, S, D):
            raise ValueError("q, k, v, out must all be [B, H, S_local, D]")
        if lse is not None and tuple(lse.shape) != (B, H, S):
            raise ValueError("lse must be [B, H, S_local]")
        mype = self.rank if rank is None else int(rank)
        # seqlens: rows held by every rank when the shards differ in length (the reference's seqlen[], csrc/ring.h:9)
        table = [S] * self.world if seqlens is None else [int(x) for x in seqlens]
        if len(table) != self.world or table[mype] != S:
            raise ValueError("seqlens must list every rank's rows and agree with this rank's tensors")
        p = set_params_fprop(q, k, v, out, self.world, mype, table, D, max(table), batch=B, heads=H, lse=lse,
                             causal=causal, softmax_scale=softmax_scale, stream=stream)
        self.forward_params(p)

    def forward_host(self, q, k, v, out, lse=None, *, chunks: int = 4, causal: bool = False,
                     softmax_scale: Optional[float] = None, stream=None, rank: Optional[int] = None) -> None:
        """Same forward with HOST tensors (pinned CPU torch tensors [B, H, S_local, D]): copies in, computes and
        copies out in `chunks` overlapping groups of (batch, head) slabs.  Asynchronous on `stream`; when the
        stream reaches the end of the call, `out` / `lse` hold the results."""
        import torch
        B, H, S, D = q.shape
        for x, n in ((q, "q"), (k, "k"), (v, "v"), (out, "out")):
            if x.is_cuda or not x.is_contiguous() or not x.is_pinned():
                raise ValueError(f"{n} must be a contiguous pinned host tensor")
            if tuple(x.shape) != (B, H, S, D):
                raise ValueError("q, k, v, out must all be [B, H, S_local, D]")
        if q.dtype not in _half_types() or out.dtype != torch.float32:
            raise ValueError("q, k, v must be fp16/bf16 and out fp32")
        if lse is not None and (lse.is_cuda or not lse.is_pinned() or tuple(lse.shape) != (B, H, S)):
            raise ValueError("lse must be a pinned host tensor [B, H, S_local]")
        mype = self.rank if rank is None else int(rank)
        p = set_params_fprop(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), self.world, mype, [S] * self.world,
                             D, S, batch=B, heads=H, lse=None if lse is None else lse.data_ptr(), causal=causal,
                             softmax_scale=softmax_scale, stream=stream)
        p.is_bf16 = int(q.dtype == torch.bfloat16)
        check(_lib.load().ring_attention_fwd_host(self._h, ctypes.byref(p), int(chunks)), "ring_attention_fwd_host")

    def synchronize(self, timeout_ms: Optional[int] = None) -> None:
        """Waits for everything the context enqueued.  With timeout_ms the wait is polled from the host and raises
        RingError (code RING_ERR_HOST_TIMEOUT) when the deadline passes; the context stays usable."""
        if timeout_ms is None:
            check(_lib.load().ring_ctx_synchronize(self._h), "ring_ctx_synchronize")
        else:
            check(_lib.load().ring_ctx_synchronize_timeout(self._h, int(timeout_ms)), "ring_ctx_synchronize_timeout")

    def timings(self):
        """(compute_ms, comm_ms, exposed_ms) lists of the last forward, one entry per ring step."""
        n = self.world
        a, b, c = ((ctypes.c_float * n)() for _ in range(3))
        check(_lib.load().ring_ctx_get_timings(self._h, a, b, c, n), "ring_ctx_get_timings")
        return list(a), list(b), list(c)

    def exchange_timings(self):
        """(wait_ms, copy_ms) lists of the last forward's exchanges, one entry per ring step: time spent waiting
        for the go-ahead, and the transfer itself."""
        n = self.world
        a, b = ((ctypes.c_float * n)() for _ in range(2))
        check(_lib.load().ring_ctx_get_exchange_timings(self._h, a, b, n), "ring_ctx_get_exchange_timings")
        return list(a), list(b)

    def abort(self) -> None:
        """After synchronize(timeout_ms=...) raised RING_ERR_HOST_TIMEOUT: release every queued wait of this context
        from the host, abort its communicator and mark it dead; destroy() then returns without waiting for the device."""
        check(_lib.load().ring_ctx_abort(self._h), "ring_ctx_abort")

    def destroy(self) -> None:
        if self._h:
            _lib.load().ring_ctx_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def attention_block_fwd(q, k, v, o, lse, *, softmax_scale: Optional[float] = None, causal: bool = False,
                        q_off: int = 0, k_off: int = 0, merge: bool = False, stream=None) -> None:
    """One Q shard [B,H,Sq,D] against one K/V shard [B,H,Sk,D] -> o [B,H,Sq,D] fp32, lse [B,H,Sq] fp32."""
    import torch
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if tuple(k.shape) != (B, H, Sk, D) or tuple(v.shape) != (B, H, Sk, D):
        raise ValueError("k, v must be [B, H, Sk, D]")
    if tuple(o.shape) != (B, H, Sq, D) or tuple(lse.shape) != (B, H, Sq):
        raise ValueError("o must be [B, H, Sq, D] and lse [B, H, Sq]")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    check(_lib.load().ring_attention_block_fwd(
        _ptr(q, "q", _half_types()), _ptr(k, "k", _half_types()), _ptr(v, "v", _half_types()),
        _ptr(o, "o", (torch.float32,)), _ptr(lse, "lse", (torch.float32,)), B, H, Sq, Sk, D, scale,
        int(bool(causal)), int(q_off), int(k_off), int(bool(merge)), int(q.dtype == torch.bfloat16),
        _stream_handle(stream)), "ring_attention_block_fwd")


def lse_merge(o_acc, lse_acc, o_part, lse_part, *, stream=None) -> None:
    """(o_acc, lse_acc) <- merge with (o_part, lse_part); tensors [..., D] fp32 and [...] fp32."""
    import torch
    D = o_acc.shape[-1]
    rows = lse_acc.numel()
    if o_acc.numel() != rows * D or o_part.numel() != rows * D or lse_part.numel() != rows:
        raise ValueError("shape mismatch between the partials")
    f32 = (torch.float32,)
    check(_lib.load().ring_lse_merge(_ptr(o_acc, "o_acc", f32), _ptr(lse_acc, "lse_acc", f32),
                                     _ptr(o_part, "o_part", f32), _ptr(lse_part, "lse_part", f32),
                                     rows, D, _stream_handle(stream)), "ring_lse_merge")


def device_status() -> int:
    s = ctypes.c_int(0)
    check(_lib.load().ring_device_status(ctypes.byref(s)), "ring_device_status")
    return s.value


def device_status_reset() -> None:
    check(_lib.load().ring_device_status_reset(), "ring_device_status_reset")


def kernel_launch_count() -> int:
    return int(_lib.load().ring_kernel_launch_count())


def attention_chunked_fwd_static(q, k, v, o, lse, kv_chunk: int, *, softmax_scale: Optional[float] = None,
                                 causal: bool = False, stream=None) -> None:
    """Attention of q [B,H,Sq,D] against k/v [B,H,Sk,D], `kv_chunk` key rows at a time, for hosts that do
    not let this library allocate device memory (a runtime that owns the whole GPU, a fixed memory budget).
    Nothing is allocated: the partial of each chunk lives in a fixed ~16 MiB array inside the library, so
    B*H*Sq <= 65536 rows and B*H*Sq*D <= 4 Mi floats, and calls that overlap on the GPU would race on it.
    The first call on a device also does the one-time set-up; make it before any stream capture."""
    import torch
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if tuple(k.shape) != (B, H, Sk, D) or tuple(v.shape) != (B, H, Sk, D):
        raise ValueError("k, v must be [B, H, Sk, D]")
    if tuple(o.shape) != (B, H, Sq, D) or tuple(lse.shape) != (B, H, Sq):
        raise ValueError("o must be [B, H, Sq, D] and lse [B, H, Sq]")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    check(_lib.load().ring_attention_chunked_fwd_static(
        _ptr(q, "q", _half_types()), _ptr(k, "k", _half_types()), _ptr(v, "v", _half_types()),
        _ptr(o, "o", (torch.float32,)), _ptr(lse, "lse", (torch.float32,)), B, H, Sq, Sk, D, scale,
        int(bool(causal)), int(kv_chunk), int(q.dtype == torch.bfloat16), _stream_handle(stream)),
        "ring_attention_chunked_fwd_static")


def static_status(stream=None) -> int:
    """Status word of the no-allocation path: waits for `stream`, then returns 0 or the code of the bounded wait that
    ran out inside the last attention_chunked_fwd_static() on this device (its outputs are then invalid)."""
    s = ctypes.c_int(0)
    check(_lib.load().ring_static_status(ctypes.byref(s), _stream_handle(stream)), "ring_static_status")
    return s.value
