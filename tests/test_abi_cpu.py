"""No-GPU checks of the boundary: the library loads, exports every declared symbol, and rejects bad
arguments with a status code before touching the device."""
import ctypes
import os
import re

import pytest

from ringattention_b200 import _lib
from ringattention_b200 import build as lib_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    lib_build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ring_attention_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ring_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SYMBOLS, f"{name} has no ctypes signature"
    assert sorted(_lib.SYMBOLS) == declared


def test_params_struct_matches_reference_prefix():
    """The first twelve fields are the reference's Ring_fwd_params (csrc/ring.h:5-19), in order."""
    names = [f[0] for f in _lib.Ring_fwd_params._fields_]
    assert names[:12] == ["mype", "npes", "seqlen", "h_seqlen", "dim", "softmax_scale", "q_ptr", "k_ptr", "v_ptr",
                          "out_ptr", "k_buffer", "v_buffer"]
    header = open(os.path.join(ROOT, "ringattention_b200", "csrc", "ring.h")).read()
    order = [header.index(" " + n + ";") if (" " + n + ";") in header else header.index("*" + n + ";") for n in names]
    assert order == sorted(order)


@pytest.mark.parametrize("kwargs,needle", [
    (dict(dim=96), "dim must be 64 or 128"),
    (dict(sq=(1 << 24) + 1), "2^24"),
    (dict(sk=0), "must be positive"),
    (dict(q=0), "null tensor pointer"),
    (dict(scale=0.0), "softmax_scale"),
    (dict(q=0x1008), "16-byte aligned"),
    (dict(batch=70000), "65535"),
])
def test_block_fwd_rejects_bad_arguments(lib, kwargs, needle):
    a = dict(q=0x1000, k=0x2000, v=0x3000, o=0x4000, lse=0x5000, batch=1, heads=1, sq=128, sk=128, dim=64, scale=0.125)
    a.update(kwargs)
    rc = lib.ring_attention_block_fwd(a["q"], a["k"], a["v"], a["o"], a["lse"], a["batch"], a["heads"], a["sq"], a["sk"],
                                      a["dim"], a["scale"], 0, 0, 0, 0, 0, None)
    assert rc == _lib.RING_ERR_INVALID_ARGUMENT
    assert needle in lib.ring_last_error_string().decode()


def test_merge_and_legacy_entry_reject_bad_arguments(lib):
    assert lib.ring_lse_merge(0x1000, 0x2000, 0x3000, 0x4000, 8, 96, None) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_lse_merge(None, 0x2000, 0x3000, 0x4000, 8, 64, None) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_lse_merge(0x1000, 0x2000, 0x3000, 0x4000, -1, 64, None) == _lib.RING_ERR_INVALID_ARGUMENT
    seqlen = (ctypes.c_int * 2)(256, 256)
    # npes > 1 without a registered context
    assert lib.ring_attention(0x1000, 0x2000, 0x3000, 0x4000, 2, 0, seqlen, 64, 256) == _lib.RING_ERR_NO_CONTEXT
    assert lib.ring_attention(0x1000, 0x2000, 0x3000, 0x4000, 2, 5, seqlen, 64, 256) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_attention(0x1000, 0x2000, 0x3000, 0x4000, 1, 0, None, 64, 256) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_attention(0x1000, 0x2000, 0x3000, 0x4000, 1, 0, seqlen, 64, 128) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_ctx_create(None, 0, 1, None) == _lib.RING_ERR_INVALID_ARGUMENT
    h = ctypes.c_void_p()
    assert lib.ring_ctx_create(ctypes.byref(h), 3, 2, None) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_ctx_create(ctypes.byref(h), 0, 2, None) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_ctx_set_option(None, 1, 1) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_get_unique_id(None) == _lib.RING_ERR_INVALID_ARGUMENT
    # the entry points added for tear-down, exchange timings and the no-allocation path's status word
    assert lib.ring_ctx_abort(None) == _lib.RING_ERR_INVALID_ARGUMENT
    f = (ctypes.c_float * 2)()
    assert lib.ring_ctx_get_exchange_timings(None, f, f, 2) == _lib.RING_ERR_INVALID_ARGUMENT
    assert lib.ring_static_status(None, None) == _lib.RING_ERR_INVALID_ARGUMENT
    assert b"null" in lib.ring_last_error_string()


def test_product_never_imports_the_oracle():
    """The shipped package must not reach into oracle/ (it is test infrastructure)."""
    pkg = os.path.join(ROOT, "ringattention_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                for pat in (r"^\s*(from|import)\s+oracle", r"liboracle", r"oracle[/\\.]oracle", r"attention_oracle"):
                    assert not re.search(pat, text, flags=re.M), f"{f} reaches into the oracle ({pat})"


def test_torch_front_end_builds_and_checks_inputs():
    """The torch extension compiles against this torch, exports its three functions, and its CHECK_INPUT
    guard rejects a CPU tensor before anything reaches the GPU library."""
    torch = pytest.importorskip("torch")
    from ringattention_b200 import build, torch_ops
    build.build_torch_ext()
    ext = torch_ops._load()
    for name in ("block_forward", "ring_forward", "lse_merge_"):
        assert callable(getattr(ext, name))
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        torch_ops.block_forward(q, q, q)
