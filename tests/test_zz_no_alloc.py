"""fa_decode_static: the decode entry point for callers that cannot allocate device memory
(a custom-call handler that only receives pre-planned buffers, a serving loop with a fixed
pool, code running under stream capture).  Its split-KV scratch is a device array inside the
library, so the caller passes inputs and outputs only.

The test drives the entry point through the C ABI and compares it with fa_decode (caller-owned
workspace) on two calls in a row with different inputs: the second call finds the first
call's leftovers in the shared scratch and must not be affected by them.  Collected last on
purpose, so a run that stops at the first failure has already run everything else."""
import ctypes as C

import pytest
import torch

from _util import max_abs, qkv

pytestmark = pytest.mark.gpu


def _problem(seed_shift, B, H, Sq, Skv, D, dtype):
    from flaxattention_b200 import attention as A
    from flaxattention_b200.masks import generate_causal_offset
    from flaxattention_b200.mods import generate_alibi_bias
    import flaxattention_b200 as fa

    q, k, v = (t.cuda() for t in qkv(B, H, H, Sq, Skv, D, dtype=dtype))
    if seed_shift:
        q, k, v = q.flip(2) * 0.5, k.flip(0) * 1.5, v.flip(1) + 1.0
    mask = generate_causal_offset(Skv - Sq)
    bm = fa.create_block_mask(mask, B, H, Sq, Skv)
    call = A._Call(q, k, v, generate_alibi_bias(H), mask, bm, D ** -0.5, "bhsd", 0, 0, None)
    return call, q, k, v


def _run_both(call, q, k, v, splits):
    from flaxattention_b200 import _cabi

    L = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        out = call.out_like(q)
        lse = torch.empty(call.B, call.Hq, call.Sq, dtype=torch.float32, device=q.device)
        p = call.params(q, k, v, out, lse)
        if static:
            _cabi.check(L.fa_decode_static(call.module.handle, C.byref(p), splits, stream))
        else:
            nbytes = L.fa_decode_workspace_bytes(C.byref(p), splits)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
            _cabi.check(L.fa_decode(call.module.handle, C.byref(p), splits, ws.data_ptr(), nbytes, stream))
        torch.cuda.synchronize()
        outs.append((out, lse))
    return outs


def test_static_scratch_decode_equals_workspace_decode_twice():
    # first call: many rows and splits; second call: a smaller problem that reuses the scratch;
    # then the 33..64-row case, where a different kernel (the tcgen05 split-KV variant) writes the
    # scratch, in bf16, again followed by a smaller problem
    cases = ((0, (2, 4, 16, 4096, 64), 6, torch.float16), (1, (1, 4, 1, 2048, 64), 3, torch.float16),
             (0, (2, 4, 48, 4096, 64), 8, torch.bfloat16), (1, (1, 2, 64, 2048, 64), 4, torch.bfloat16))
    for shift, shape, splits, dtype in cases:
        call, q, k, v = _problem(shift, *shape, dtype)
        (o_ws, l_ws), (o_st, l_st) = _run_both(call, q, k, v, splits)
        assert not torch.isnan(o_st.float()).any()
        assert max_abs(o_st, o_ws) <= 2e-3
        assert max_abs(l_st, l_ws) <= 2e-3 * max(1.0, l_ws.abs().max().item())


def test_static_scratch_rejects_oversized_problems():
    from flaxattention_b200 import _cabi

    L = _cabi.lib()
    cap = L.fa_decode_static_capacity()
    assert 1 << 20 <= cap <= 64 << 20
    call, q, k, v = _problem(0, 8, 8, 64, 1024, 64, torch.float16)
    out = call.out_like(q)
    p = call.params(q, k, v, out, None)
    splits = 64
    assert L.fa_decode_workspace_bytes(C.byref(p), splits) > cap
    rc = L.fa_decode_static(call.module.handle, C.byref(p), splits, torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    msg = L.fa_last_error().decode()
    assert str(cap) in msg and "scratch" in msg


def test_static_scratch_validates_before_sizing():
    """Bad shapes are argument errors (FA_EINVAL), whatever their product would be as a size."""
    from flaxattention_b200 import _cabi

    L = _cabi.lib()
    call, q, k, v = _problem(0, 1, 2, 4, 1024, 64, torch.float16)
    out = call.out_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    for field, value in (("B", -1), ("Sq", 0), ("Hq", -4)):
        p = call.params(q, k, v, out, None)
        setattr(p, field, value)
        assert L.fa_decode_static(call.module.handle, C.byref(p), 4, stream) == -1, field
