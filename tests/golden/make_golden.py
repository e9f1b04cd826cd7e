"""Generate the golden fixtures in this directory by EXECUTING the reference's own
attention statements (csrc/self_attention.py:22-26 of ykcombat/RingAttention) on CPU.

The reference script builds its tensors on "cuda" and runs at import, so it cannot be
imported here.  This generator reads the script as text, takes exactly the three compute
statements of its loop body (scores / weights / output, lines 22, 23 and 26), and execs
them, unmodified, in a namespace whose Q, K, V are CPU tensors:
  * fp64-widened copies of seeded fp16 inputs  -> `o_f64` (the golden output) and
    `lse_f64` = logsumexp of the reference's own `scores` variable;
  * the fp16 tensors themselves, as the reference runs them -> `o_f16` (loose check).
The reference has no softmax scale (it is 1).  A scale of 2^-3 is obtained by
pre-multiplying Q by 0.125 (exactly, in fp64) before the reference statements run.

Run from the repository root with the path of a checkout of the reference (the fixtures travel, it does not):
    python tests/golden/make_golden.py <path to ykcombat/RingAttention>
"""
import os
import sys
import textwrap

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from ringattention_b200 import synthetic  # noqa: E402

CASES = [
    # name, seed, S, D, q_prescale (=softmax scale), gain
    ("ref_s256_d64_scale1", 11, 256, 64, 1.0, 0.5),
    ("ref_s256_d64_scale0125", 12, 256, 64, 0.125, 1.0),
    ("ref_s384_d128_scale0125", 13, 384, 128, 0.125, 1.0),
]


def reference_statements(ref_root: str) -> str:
    path = os.path.join(ref_root, "csrc", "self_attention.py")
    lines = open(path, encoding="utf-8").read().splitlines()
    picked = [lines[i - 1] for i in (22, 23, 26)]
    src = textwrap.dedent("\n".join(picked))
    assert "torch.matmul(Q, K.transpose(0, 1))" in src and "F.softmax(scores, dim=-1)" in src \
        and "torch.matmul(weights, V)" in src, "reference statements moved; check line numbers"
    return src


def run_reference(src: str, Q, K, V):
    ns = {"torch": torch, "F": F, "Q": Q, "K": K, "V": V}
    exec(compile(src, "reference:csrc/self_attention.py:22-26", "exec"), ns)
    return ns["scores"], ns["output"]


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    ref_root = sys.argv[1]
    src = reference_statements(ref_root)
    for name, seed, S, D, prescale, gain in CASES:
        q, k, v = synthetic.make_qkv(seed, 1, 1, D, 0, S, gain)
        q2, k2, v2 = (torch.from_numpy(x[0, 0].copy()) for x in (q, k, v))
        # The fp64 run scales Q exactly; the fp16 run rounds the few subnormal products.
        qs = (q2 * prescale).to(torch.float16)
        scores, out64 = run_reference(src, q2.double() * prescale, k2.double(), v2.double())
        lse64 = torch.logsumexp(scores, dim=-1)
        _, out16 = run_reference(src, qs, k2, v2)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            q=q[0, 0], k=k[0, 0], v=v[0, 0], scale=np.float64(prescale), seed=np.int64(seed),
            gain=np.float64(gain), o_f64=out64.numpy().astype(np.float32),
            lse_f64=lse64.numpy().astype(np.float32), o_f16=out16.numpy().astype(np.float16))
        print(name, "written; |o|max", float(out64.abs().max()))


if __name__ == "__main__":
    main()
