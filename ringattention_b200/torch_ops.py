"""torch.Tensor front end: the operator the reference's include/attention_api.cuh:1-30 prepares for
(torch/extension.h plus the CHECK_INPUT argument checks) but never declares.

The functions here take and return torch tensors; argument checking (CUDA device, contiguity, dtype, shape)
happens in C++ (csrc/torch_ext.cpp) with the reference's CHECK_INPUT macro, the work happens in the C-ABI
library.  The extension is compiled by ``python -m ringattention_b200.build --torch``; importing this module
without it raises, there is no fallback.  Forward only, as in the reference.
"""
from __future__ import annotations

import importlib
from typing import Optional, Sequence, Tuple

_ext = None


def _load():
    global _ext
    if _ext is None:
        import torch  # noqa: F401  (the extension resolves libtorch symbols from the loaded torch)
        try:
            _ext = importlib.import_module("ringattention_b200._torch_ext")
        except ImportError as e:
            raise ImportError("ringattention_b200._torch_ext is not built: run "
                              "`python -m ringattention_b200.build --torch`") from e
    return _ext


def block_forward(q, k, v, softmax_scale: Optional[float] = None, causal: bool = False, q_off: int = 0, k_off: int = 0) -> Tuple:
    """One Q shard [B,H,Sq,D] against one K/V shard [B,H,Sk,D] (fp16 or bf16): returns (out fp32, lse fp32).

    The flash inner loop over one source shard and the final normalisation (csrc/ring_attention.cu:536-609,
    621-664).  softmax_scale None means 1/sqrt(D); q_off / k_off place the shards in the global sequence for the
    causal mask.  Asynchronous on the current torch stream.
    """
    return tuple(_load().block_forward(q, k, v, float(softmax_scale or 0.0), bool(causal), int(q_off), int(k_off)))


def ring_forward(ctx, q, k, v, seqlens: Optional[Sequence[int]] = None, softmax_scale: Optional[float] = None,
                 causal: bool = False, mype: Optional[int] = None) -> Tuple:
    """Ring-attention forward of this rank through a RingContext: returns (out fp32, lse fp32).

    set_params_fprop + run_ring_fwd of the reference (csrc/ring_attention.cu:361-395, 669-704) on tensors.
    seqlens are the rows of every rank's shard (default: all equal to this rank's); mype defaults to ctx.rank
    (virtual-rank contexts pass it explicitly).  Asynchronous on the current torch stream.
    """
    rank = ctx.rank if mype is None else int(mype)
    lens = [int(q.shape[2])] * ctx.world if seqlens is None else [int(s) for s in seqlens]
    return tuple(_load().ring_forward(int(ctx._h.value), q, k, v, lens, rank, float(softmax_scale or 0.0), bool(causal)))


def lse_merge_(o_acc, lse_acc, o_part, lse_part) -> None:
    """Merges the partial (o_part, lse_part) into (o_acc, lse_acc) in place (csrc/ring_attention.cu:439-443, 621-633)."""
    _load().lse_merge_(o_acc, lse_acc, o_part, lse_part)
