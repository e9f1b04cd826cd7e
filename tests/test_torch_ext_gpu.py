"""The torch.Tensor front end (csrc/torch_ext.cpp) against the CPU oracle, and its argument checks."""
import numpy as np
import pytest

from tests.gpu_util import assert_parity

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ringattention_b200 import build, torch_ops
    build.build_torch_ext()
    torch_ops._load()
    return torch_ops


def _qkv(seed, b, h, s, d):
    from ringattention_b200 import synthetic
    return synthetic.make_qkv(seed, b, h, d, 0, s)


@pytest.mark.parametrize("causal", [False, True])
def test_block_forward_matches_oracle(ops, causal):
    from oracle import oracle
    q, k, v = _qkv(11, 1, 2, 512, 128)
    dev = torch.device("cuda:0")
    out, lse = ops.block_forward(torch.from_numpy(q).to(dev), torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev),
                                 causal=causal)
    ref_o, ref_l = oracle.attention_fwd(q, k, v, 1.0 / np.sqrt(128), causal=causal)
    assert_parity(out.cpu().numpy(), lse.cpu().numpy(), ref_o, ref_l)


def test_ring_forward_virtual_ranks(ops):
    from oracle import oracle
    from ringattention_b200 import RingContext
    world, s_loc, d = 2, 256, 64
    q, k, v = _qkv(12, 1, 2, world * s_loc, d)
    dev = torch.device("cuda:0")
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
    shard = lambda t, r: t[:, :, r * s_loc:(r + 1) * s_loc].contiguous()
    ks, vs = [shard(tk, r) for r in range(world)], [shard(tv, r) for r in range(world)]
    ctx = RingContext.create_local(world)
    try:
        ctx.set_local_shards(ks, vs)
        ref_o, ref_l = oracle.attention_fwd(q, k, v, 1.0 / np.sqrt(d), causal=True)
        for r in range(world):
            out, lse = ops.ring_forward(ctx, shard(tq, r), ks[r], vs[r], causal=True, mype=r)
            ctx.synchronize()
            assert_parity(out.cpu().numpy(), lse.cpu().numpy(), ref_o[:, :, r * s_loc:(r + 1) * s_loc],
                          ref_l[:, :, r * s_loc:(r + 1) * s_loc])
    finally:
        ctx.destroy()


def test_merge_of_two_halves_equals_whole(ops):
    q, k, v = _qkv(13, 1, 1, 512, 128)
    dev = torch.device("cuda:0")
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
    whole_o, whole_l = ops.block_forward(tq, tk, tv)
    o_a, l_a = ops.block_forward(tq, tk[:, :, :256].contiguous(), tv[:, :, :256].contiguous())
    o_b, l_b = ops.block_forward(tq, tk[:, :, 256:].contiguous(), tv[:, :, 256:].contiguous(), k_off=256)
    ops.lse_merge_(o_a, l_a, o_b, l_b)
    assert torch.max(torch.abs(o_a - whole_o)).item() <= 2e-3
    assert torch.max(torch.abs(l_a - whole_l)).item() <= 1e-4


def test_check_input_rejects(ops):
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device=dev)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ops.block_forward(q.cpu(), q, q)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        ops.block_forward(q, q[:, :, ::2], q[:, :, ::2])
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        ops.block_forward(q.float(), q.float(), q.float())
    with pytest.raises(RuntimeError, match="failed"):
        ops.block_forward(q[..., :48].contiguous(), q[..., :48].contiguous(), q[..., :48].contiguous())
