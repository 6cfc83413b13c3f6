"""Host-side checks of the C ABI that need no GPU: the library loads, exports every symbol
include/flaxattn.h declares, and rejects bad arguments before touching CUDA."""
import ctypes as C
import os
import re

import pytest

from flaxattention_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    out = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            out.update(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text))
    return out


def test_library_exports_every_declared_symbol():
    L = _cabi.lib()
    syms = _declared_symbols()
    assert len(syms) >= 16
    for s in syms:
        assert hasattr(L, s), f"{s} is declared in include/ but not exported"
    assert syms >= set(_cabi.EXPORTS)
    assert L.fa_version() >= 100


def _params(**kw):
    p = _cabi.FaAttnParams()
    p.dtype, p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.D, p.Dv = 0, 1, 2, 2, 64, 64, 64, 64
    p.scale = 0.125
    for t in ("q", "k", "v", "o"):
        getattr(p, t).ptr = 0x1000
        getattr(p, t).stride_b, getattr(p, t).stride_h, getattr(p, t).stride_s = 2 * 64 * 64, 64 * 64, 64
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,code,frag", [
    (dict(D=60, Dv=60), -4, "multiples of 16"),
    (dict(Hkv=3), -1, "multiple of Hkv"),
    (dict(Dv=128), -1, "must not exceed"),
    (dict(dtype=7), -1, "dtype"),
    (dict(Sq=0), -1, "positive"),
    (dict(D=512, Dv=64), -4, "256"),
])
def test_argument_validation(kw, code, frag):
    L = _cabi.lib()
    m = _cabi.Module(None)
    rc = L.fa_fwd(m.handle, C.byref(_params(**kw)), None)
    assert rc == code
    assert frag in L.fa_last_error().decode()


def test_pointer_and_stride_validation():
    L = _cabi.lib()
    m = _cabi.Module(None)
    p = _params()
    p.k.ptr = None
    assert L.fa_fwd(m.handle, C.byref(p), None) == -1 and "k: null" in L.fa_last_error().decode()
    p = _params()
    p.v.ptr = 0x1004
    assert L.fa_fwd(m.handle, C.byref(p), None) == -1 and "aligned" in L.fa_last_error().decode()
    p = _params()
    p.q.stride_s = 65
    assert L.fa_fwd(m.handle, C.byref(p), None) == -1 and "strides" in L.fa_last_error().decode()
    assert L.fa_fwd(None, C.byref(_params()), None) == -1


def test_block_table_validation():
    L = _cabi.lib()
    m = _cabi.Module(None)
    p = _params()
    p.tables.kv_num_blocks = 0x2000
    p.tables.kv_indices = 0x3000
    p.tables.mask_B = p.tables.mask_H = 1
    p.tables.num_q_blocks = p.tables.num_kv_blocks = 1
    p.tables.q_block_size = p.tables.kv_block_size = 32  # covers 32 < 64 tokens
    assert L.fa_fwd(m.handle, C.byref(p), None) == -1
    assert "cover" in L.fa_last_error().decode()
    p.tables.q_block_size = p.tables.kv_block_size = 128
    p.tables.mask_H = 3
    assert L.fa_fwd(m.handle, C.byref(p), None) == -1


def test_workspace_queries_and_checks():
    L = _cabi.lib()
    m = _cabi.Module(None)
    p = _params(B=2, Hq=4, Hkv=4, Sq=16, Skv=4096)
    assert L.fa_bwd_workspace_bytes(C.byref(p)) >= 2 * 4 * 16 * 4
    assert L.fa_decode_workspace_bytes(C.byref(p), 1) == 0
    assert L.fa_decode_workspace_bytes(C.byref(p), 4) >= 2 * 4 * 4 * 16 * (64 + 2) * 4
    assert 1 <= L.fa_decode_num_splits(C.byref(p), 148) <= 256
    assert L.fa_decode(m.handle, C.byref(p), 4, None, 0, None) == -5
    p.lse = 0x4000
    t = _cabi.FaTensor(0x5000, 1, 1, 64)
    t.stride_b, t.stride_h = 4 * 16 * 64, 16 * 64
    assert L.fa_bwd(m.handle, C.byref(p), C.byref(t), C.byref(t), C.byref(t), C.byref(t), None, 0, None) == -5
    assert L.fa_block_mask_workspace_bytes(2, 3, 200, 300, 128, 128) == 2 * 3 * 2 * 3
    assert L.fa_block_mask(m.handle, 1, 1, 64, 64, 64, 64, 0, 0, *([None] * 8), None, 0, None) == -1


def test_product_fails_loudly_without_cuda():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import flaxattention_b200 as fa

    q = torch.zeros(1, 1, 16, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        fa.flax_attention(q, q, q)
    with pytest.raises(RuntimeError, match="CUDA"):
        fa.create_block_mask(fa.masks.causal_mask, 1, 1, 128, 128)


def test_reference_validation_messages():
    """Error behaviour of the reference's entry points (core/attention.py:119-198)."""
    import torch
    import flaxattention_b200 as fa

    q = torch.zeros(1, 4, 16, 16)
    with pytest.raises(ValueError, match="same dtype"):
        fa.flax_attention(q, q.half(), q)
    with pytest.raises(ValueError, match="same number of heads"):
        fa.flax_attention(q, q[:, :2], q[:, :2])
    with pytest.raises(ValueError, match="multiple of kv heads"):
        fa.flax_attention(q, q[:, :3], q[:, :3], enable_gqa=True)
    with pytest.raises(ValueError, match="embedding dimension"):
        fa.flax_attention(q, q[..., :8], q)
    with pytest.raises(NotImplementedError, match="4D"):
        fa.flax_attention(q[0], q[0], q[0])
    with pytest.raises(ValueError, match="same number of heads"):
        fa.flax_attention_pallas(q, q[:, :2], q[:, :2])


def test_decode_static_rejects_bad_arguments_first():
    """fa_decode_static validates before it sizes its scratch: negative or zero extents are
    FA_EINVAL, not a workspace error with a wrapped-around byte count."""
    L = _cabi.lib()
    m = _cabi.Module(None)
    for kw in (dict(B=-2), dict(Sq=0), dict(Hq=-4, Hkv=-4)):
        assert L.fa_decode_static(m.handle, C.byref(_params(Skv=4096, **kw)), 4, None) == -1, kw
    assert L.fa_decode_static(m.handle, C.byref(_params(Sq=65, Skv=4096)), 4, None) == -4
    assert L.fa_decode_static(m.handle, C.byref(_params(dtype=2, Sq=8, Skv=4096)), 4, None) == -4
    assert L.fa_decode_static(m.handle, None, 4, None) == -1


def test_status_word_raises_on_the_next_check():
    """A kernel that gave up on a barrier wait ORs a bit into the status word; the wrapper raises
    on the next call or on check_status() and clears the word."""
    import torch
    from flaxattention_b200 import attention as A

    old = A._status_word
    try:
        A._status_word = torch.zeros(1, dtype=torch.int32)
        A.check_status()
        A._status_word[0] = 1
        with pytest.raises(_cabi.FlaxAttnError, match="barrier wait"):
            A.check_status()
        A.check_status()  # cleared
    finally:
        A._status_word = old


def test_profile_read_without_a_call_is_empty():
    L = _cabi.lib()
    assert L.fa_profile_enable(1) == 0
    assert _cabi.profile_read() == []
    assert L.fa_profile_enable(0) == 0


def test_other_buffers_are_bound_as_trailing_arguments():
    """math_attention(..., score_mod_other_buffers, mask_mod_other_buffers): the reference calls
    the mods with the buffers appended (core/attention.py:35-52)."""
    import torch
    from flaxattention_b200 import attention as A, modtrace

    bias = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    doc = torch.tensor([0, 0, 1, 1], dtype=torch.int32)

    def score(s, b, h, q, kv, table):
        return s + table[h, kv]

    def mask(b, h, q, kv, ids):
        return ids[q] == ids[kv]

    sb = A._bind_other_buffers(score, (bias,), True)
    mb = A._bind_other_buffers(mask, (doc,), False)
    assert A._bind_other_buffers(score, (bias,), True) is sb  # cached on identity
    assert modtrace.mod_arity(sb) == 5 and modtrace.mod_arity(mb) == 4
    ms = modtrace.lower_mods(sb, mb)
    assert len(ms.buffers) == 2
    import numpy as np
    b = np.zeros((1, 1, 1, 1), np.int32)
    h = np.arange(3, dtype=np.int32).reshape(1, 3, 1, 1)
    q = np.arange(4, dtype=np.int32).reshape(1, 1, 4, 1)
    kv = np.arange(4, dtype=np.int32).reshape(1, 1, 1, 4)
    got = modtrace.evaluate(modtrace.trace_score_mod(sb), np.zeros((1, 3, 4, 4), np.float32), b, h, q, kv)
    assert np.array_equal(np.broadcast_to(got, (1, 3, 4, 4))[0, :, 0, :], bias.numpy())
    gm = modtrace.evaluate(modtrace.trace_mask_mod(mb), None, b, h, q, kv)
    assert np.array_equal(np.broadcast_to(gm, (1, 1, 4, 4))[0, 0], doc.numpy()[:, None] == doc.numpy()[None, :])


def test_decode_head_packing_rule():
    """fa_decode_packs_heads: grouped-query heads are packed when the rows fit one tile and the
    tables do not depend on the head."""
    L = _cabi.lib()
    p = _params(Hq=8, Hkv=2, Sq=4, Skv=4096)
    assert L.fa_decode_packs_heads(C.byref(p)) == 1
    assert L.fa_decode_packs_heads(C.byref(_params(Hq=8, Hkv=2, Sq=32, Skv=4096))) == 0   # 4 * 32 rows > 64
    assert L.fa_decode_packs_heads(C.byref(_params(Hq=4, Hkv=4, Sq=4, Skv=4096))) == 0    # not grouped
    p.tables.kv_num_blocks, p.tables.kv_indices = 0x2000, 0x3000
    p.tables.mask_B, p.tables.mask_H = 1, 8
    assert L.fa_decode_packs_heads(C.byref(p)) == 0                                          # per-head tables
    p.tables.mask_H = 1
    assert L.fa_decode_packs_heads(C.byref(p)) == 1
    assert L.fa_decode_packs_heads(None) == 0
