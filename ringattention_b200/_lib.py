"""ctypes binding of libringattn_b200.so.  There is no fallback: if the CUDA library is
missing or a symbol is absent, importing the binding raises."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libringattn_b200.so")

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

RING_OK = 0
RING_ERR_INVALID_ARGUMENT = -1
RING_ERR_CUDA = -2
RING_ERR_NCCL = -3
RING_ERR_DEVICE_TIMEOUT = -4
RING_ERR_NO_CONTEXT = -5
RING_ERR_UNSUPPORTED = -6
RING_ERR_HOST_TIMEOUT = -7
RING_UNIQUE_ID_BYTES = 128
RING_MERGE_SEPARATE_KERNEL = 0
RING_MERGE_FUSED_EPILOGUE = 1
RING_OPT_MERGE_MODE = 1
RING_OPT_CAUSAL_SKIP_EXCHANGE = 2
RING_OPT_RECORD_TIMINGS = 3
RING_OPT_TRANSPORT = 4
RING_OPT_CAUSAL_ZIGZAG = 5
RING_OPT_RECV_BUFFERS = 6
RING_TRANSPORT_NCCL = 0
RING_TRANSPORT_PEER_COPY = 1
RING_STATIC_MAX_ROWS = 65536
RING_STATIC_MAX_OUT_ELEMS = 4 * 1024 * 1024


class Ring_fwd_params(ctypes.Structure):
    """Mirror of csrc/ring.h in this repository (the reference's struct, csrc/ring.h:5-19, first)."""
    _fields_ = [
        ("mype", c_int), ("npes", c_int),
        ("seqlen", ctypes.POINTER(c_int)), ("h_seqlen", ctypes.POINTER(c_int)),
        ("dim", c_int), ("softmax_scale", c_float),
        ("q_ptr", c_void_p), ("k_ptr", c_void_p), ("v_ptr", c_void_p), ("out_ptr", c_void_p),
        ("k_buffer", c_void_p), ("v_buffer", c_void_p),
        ("batch", c_int), ("heads", c_int), ("lse_ptr", c_void_p),
        ("causal", c_int), ("is_bf16", c_int), ("stream", c_void_p),
    ]


class RingStepPlan(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("src_rank", "compute", "compute_buffer", "recv_buffer", "recv_from", "send_to",
                                     "do_recv", "do_send")]


# name -> (restype, argtypes); every symbol declared in include/ring_attention_b200.h
SYMBOLS = {
    "ring_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(c_int), c_int, c_int]),
    "ring_attention_scaled": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(c_int), c_int, c_int, c_float]),
    "ring_get_unique_id": (c_int, [c_void_p]),
    "ring_ctx_create": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "ring_ctx_destroy": (c_int, [c_void_p]),
    "ring_ctx_set_option": (c_int, [c_void_p, c_int, c_int]),
    "ring_ctx_get_option": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int)]),
    "ring_set_default_ctx": (c_int, [c_void_p]),
    "ring_ctx_create_local": (c_int, [ctypes.POINTER(c_void_p), c_int]),
    "ring_ctx_set_local_shards": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p)]),
    "ring_attention_fwd": (c_int, [c_void_p, ctypes.POINTER(Ring_fwd_params)]),
    "ring_attention_fwd_host": (c_int, [c_void_p, ctypes.POINTER(Ring_fwd_params), c_int]),
    "ring_ctx_synchronize": (c_int, [c_void_p]),
    "ring_ctx_synchronize_timeout": (c_int, [c_void_p, c_int]),
    "ring_step_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(RingStepPlan)]),
    "ring_ctx_get_timings": (c_int, [c_void_p, ctypes.POINTER(c_float), ctypes.POINTER(c_float), ctypes.POINTER(c_float), c_int]),
    "ring_ctx_get_exchange_timings": (c_int, [c_void_p, ctypes.POINTER(c_float), ctypes.POINTER(c_float), c_int]),
    "ring_ctx_abort": (c_int, [c_void_p]),
    "ring_static_status": (c_int, [ctypes.POINTER(c_int), c_void_p]),
    "ring_attention_block_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_float, c_int, c_int64, c_int64, c_int, c_int, c_void_p]),
    "ring_lse_merge": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "ring_attention_chunked_fwd_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                  c_float, c_int, c_int, c_int, c_void_p]),
    "ring_device_status": (c_int, [ctypes.POINTER(c_int)]),
    "ring_device_status_reset": (c_int, []),
    "ring_device_status_inject": (c_int, [c_int]),
    "ring_selftest_wait_timeout": (c_int, [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_float)]),
    "ring_kernel_launch_count": (c_int64, []),
    "ring_last_error_string": (ctypes.c_char_p, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ringattention_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


class RingError(RuntimeError):
    def __init__(self, code: int, where: str):
        msg = load().ring_last_error_string()
        super().__init__(f"{where} failed with status {code}: {msg.decode() if msg else ''}")
        self.code = code


def check(code: int, where: str) -> None:
    if code != RING_OK:
        raise RingError(code, where)
