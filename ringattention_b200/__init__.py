"""B200-native ring-attention forward (drop-in for the hot path of ykcombat/RingAttention).

The package holds the host-side mirror of the reference's operator interface (api.py), the C-ABI
binding (_lib.py), the build recipe (build.py), the seeded synthetic inputs (synthetic.py) and the
CUDA sources (csrc/).  Importing it does not load the CUDA library; the first call does, and fails
loudly if the library has not been built.
"""
from .api import (Ring_fwd_params, RingContext, attention_block_fwd, attention_chunked_fwd_static, device_status, device_status_reset,
                  kernel_launch_count, lse_merge, ring_attention, ring_attention_scaled, set_params_fprop, static_status)
from ._lib import (RING_MERGE_FUSED_EPILOGUE, RING_MERGE_SEPARATE_KERNEL, RING_OPT_CAUSAL_SKIP_EXCHANGE,
                   RING_OPT_MERGE_MODE, RING_OPT_RECORD_TIMINGS, RING_OPT_TRANSPORT, RING_OPT_CAUSAL_ZIGZAG, RING_OPT_RECV_BUFFERS, RING_TRANSPORT_NCCL,
                   RING_TRANSPORT_PEER_COPY, RING_ERR_HOST_TIMEOUT, RingError)

__all__ = [
    "Ring_fwd_params", "RingContext", "attention_block_fwd", "attention_chunked_fwd_static", "device_status", "device_status_reset",
    "kernel_launch_count", "lse_merge", "ring_attention", "ring_attention_scaled", "set_params_fprop", "static_status",
    "RING_MERGE_FUSED_EPILOGUE", "RING_MERGE_SEPARATE_KERNEL", "RING_OPT_CAUSAL_SKIP_EXCHANGE",
    "RING_OPT_MERGE_MODE", "RING_OPT_RECORD_TIMINGS", "RING_OPT_TRANSPORT", "RING_OPT_CAUSAL_ZIGZAG", "RING_OPT_RECV_BUFFERS", "RING_TRANSPORT_NCCL",
    "RING_TRANSPORT_PEER_COPY", "RING_ERR_HOST_TIMEOUT", "RingError",
]
