"""GPU parity of the attention backward.  The bar is the one the task states: gradients
within 5e-2 of an fp32 reference, relative (max |g - ref| / max |ref|).  The fp32 reference
is the oracle with inputs upcast to fp32 and differentiated by autograd; fp32 inputs are
held to 1e-4."""
import os

import numpy as np
import pytest
import torch

from _util import DTYPES, max_abs, qkv, rel_err
from oracle.attention_oracle import attention_grads_oracle

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ATT = np.load(os.path.join(HERE, "golden", "attention_golden.npz"))
GTOL = {"f16": 5e-2, "bf16": 5e-2, "f32": 1e-4}


def _grads(q, k, v, dout, score_mod, mask_mod, block_size=128, **kw):
    import flaxattention_b200 as fa

    B, Hq, Sq, _ = q.shape
    Skv = k.shape[2]
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bm = fa.create_block_mask(mask_mod, B, Hq, Sq, Skv, BLOCK_SIZE=block_size) if mask_mod is not None else None
    out = fa.flax_attention(qc, kc, vc, score_mod=score_mod, block_mask=bm, enable_gqa=q.shape[1] != k.shape[1],
                            kernel_options={"path": "fwd"}, **kw)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    return out.detach().cpu(), qc.grad.cpu(), kc.grad.cpu(), vc.grad.cpu()


CASES = [
    # B, Hq, Hkv, Sq, Skv, D, Dv, dtype, score, mask, block
    (2, 4, 4, 64, 64, 32, 32, "f32", None, None, 128),
    (2, 4, 4, 256, 256, 64, 64, "f32", "alibi", "causal", 128),       # the CPU-runnable configuration
    (2, 4, 4, 256, 256, 64, 64, "f16", "checker", None, 128),
    (1, 4, 4, 512, 512, 64, 64, "bf16", "alibi", "causal", 128),
    (1, 2, 2, 1024, 1024, 128, 128, "bf16", None, "sink", 128),
    (1, 4, 2, 200, 333, 64, 64, "f16", "alibi", "causal", 128),        # ragged + GQA
    (1, 2, 2, 384, 640, 32, 32, "bf16", "softcap", "window", 64),
    (1, 2, 2, 1, 300, 64, 64, "f16", "alibi", None, 128),               # decode-shaped
    (1, 2, 2, 128, 128, 128, 64, "f32", "checker", "causal", 128),
    (1, 1, 1, 320, 320, 256, 256, "f16", None, "causal", 128),
]


def _mods(score, mask, Hq, Sq, Skv):
    from flaxattention_b200 import fnp
    from flaxattention_b200.masks import causal_mask, generate_attention_sink, generate_sliding_window
    from flaxattention_b200.mods import checkerboard, generate_alibi_bias

    def softcap(s, b, h, q, kv):
        return 20.0 * fnp.tanh(s / 20.0)

    s = {None: None, "alibi": generate_alibi_bias(Hq), "checker": checkerboard, "softcap": softcap}[score]
    m = {None: None, "causal": causal_mask, "sink": generate_attention_sink(200, 4),
         "window": generate_sliding_window(100)}[mask]
    return s, m


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_gradients_match_fp32_reference(case):
    B, Hq, Hkv, Sq, Skv, D, Dv, dt, score, mask, bs = case
    s, m = _mods(score, mask, Hq, Sq, Skv)
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, Dv, dtype=DTYPES[dt])
    g = np.random.Generator(np.random.Philox(7))
    dout = torch.from_numpy(g.standard_normal((B, Hq, Sq, Dv), dtype=np.float32)).to(DTYPES[dt])
    out, dq, dk, dv = _grads(q, k, v, dout, s, m, bs)
    _, _, rq, rk, rv = attention_grads_oracle(q, k, v, dout, s, m)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        assert not torch.isnan(got.float()).any(), name
        assert rel_err(got, ref) <= GTOL[dt], f"{name}: {rel_err(got, ref)}"


TC_CASES = [
    # shapes the single-pass tcgen05 backward covers (D = 64): B, Hq, Hkv, Sq, Skv, dtype, score, mask
    (1, 1, 1, 128, 128, "f16", None, None),
    (2, 2, 2, 512, 512, "bf16", "checker", None),
    (1, 4, 4, 1024, 1024, "f16", "alibi", "causal"),
    (1, 2, 2, 300, 333, "f16", "alibi", "causal"),
    (1, 4, 2, 512, 768, "f16", "softcap", "window"),
    (1, 2, 2, 2048, 2048, "bf16", None, "sink"),
]


@pytest.mark.parametrize("case", TC_CASES, ids=lambda c: "-".join(map(str, c)))
def test_tcgen05_and_general_backward_agree_with_the_reference(case):
    import flaxattention_b200 as fa

    B, Hq, Hkv, Sq, Skv, dt, score, mask = case
    s, m = _mods(score, mask, Hq, Sq, Skv)
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, 64, dtype=DTYPES[dt])
    g = np.random.Generator(np.random.Philox(11))
    dout = torch.from_numpy(g.standard_normal((B, Hq, Sq, 64), dtype=np.float32)).to(DTYPES[dt])
    _, _, rq, rk, rv = attention_grads_oracle(q, k, v, dout, s, m)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = []
    for opts in ({"status": status}, {"kernels": "general"}):
        bm = fa.create_block_mask(m, B, Hq, Sq, Skv) if m is not None else None
        qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
        out = fa.flax_attention(qc, kc, vc, score_mod=s, block_mask=bm, enable_gqa=Hq != Hkv,
                                kernel_options=dict(opts, path="fwd"))
        out.backward(dout.cuda())
        torch.cuda.synchronize()
        got = (qc.grad.cpu(), kc.grad.cpu(), vc.grad.cpu())
        for name, x, r in zip(("dq", "dk", "dv"), got, (rq, rk, rv)):
            assert not torch.isnan(x.float()).any(), name
            assert rel_err(x, r) <= GTOL[dt], f"{name}: {rel_err(x, r)}"
        res.append(got)
    assert int(status.item()) == 0
    for a, b in zip(*res):
        assert rel_err(a, b) <= (4e-3 if dt == "f16" else 3e-2)


@pytest.mark.parametrize("name", ["grads_nomod", "grads_decode"])
def test_gradients_match_stored_sdpa_vectors(name):
    # tests/attention_test.py:385-477: dQ of output.sum() against torch autograd
    B, Hq, Hkv, Sq, Skv, D, _ = (int(x) for x in ATT[f"{name}.shape"])
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D)
    out, dq, dk, dv = _grads(q, k, v, torch.ones(B, Hq, Sq, D), None, None)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert max_abs(got, torch.from_numpy(ATT[f"{name}.{key}"])) <= 2e-5, key


def test_pallas_entry_point_gradient():
    # tests/attention_test.py:432-477 (test_pallas_autograd_equivalence_with_torch): dQ of
    # output.sum() through the fused entry point against the stored torch-autograd vector
    import flaxattention_b200 as fa

    B, Hq, Hkv, Sq, Skv, D, _ = (int(x) for x in ATT["grads_nomod.shape"])
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D)
    qc = q.cuda().requires_grad_(True)
    fa.flax_attention_pallas(qc, k.cuda(), v.cuda()).sum().backward()
    assert max_abs(qc.grad.cpu(), torch.from_numpy(ATT["grads_nomod.dq"])) <= 2e-5
    q, k, v = qkv(4, 8, 8, 64, 64, 32)
    qc = q.cuda().requires_grad_(True)
    fa.flax_attention_pallas(qc, k.cuda(), v.cuda()).sum().backward()
    _, _, rq, _, _ = attention_grads_oracle(q, k, v, torch.ones(4, 8, 64, 32))
    assert max_abs(qc.grad.cpu(), rq) <= 2e-5


def test_fully_masked_rows_have_zero_gradient():
    """Rows without a visible key: the dense reference yields NaN there; the kernels define
    the gradient as 0 and keep the other rows exact."""
    import flaxattention_b200 as fa

    def late_start(b, h, q, kv):
        return (q >= 64) & (q >= kv)

    q, k, v = qkv(1, 2, 2, 256, 256, 64, dtype=torch.float16)
    dout = torch.ones(1, 2, 256, 64, dtype=torch.float16)
    out, dq, dk, dv = _grads(q, k, v, dout, None, late_start)
    assert torch.count_nonzero(dq[:, :, :64]) == 0 and torch.count_nonzero(out[:, :, :64]) == 0
    _, _, rq, rk, rv = attention_grads_oracle(q, k, v, dout, None, late_start)
    assert rel_err(dq, rq) <= 5e-2 and rel_err(dk, rk) <= 5e-2 and rel_err(dv, rv) <= 5e-2


def test_benchmark_shape_backward_properties():
    """Full-size configuration (B8 H8 S2048 D64 fp16, checkerboard, dO = 1): a slice of heads
    is compared with the fp32 reference; in addition sum_q dQ.Q = sum_kv dK.K per (b, h),
    because both equal sum(dS * S) for the bilinear score, and the run is deterministic."""
    import flaxattention_b200 as fa
    from flaxattention_b200.mods import checkerboard

    q, k, v = qkv(8, 8, 8, 2048, 2048, 64, dtype=torch.float16)
    dout = torch.ones(8, 8, 2048, 64, dtype=torch.float16)
    out, dq, dk, dv = _grads(q, k, v, dout, checkerboard, None)
    sl = (slice(0, 1), slice(0, 2))
    _, _, rq, rk, rv = attention_grads_oracle(q[sl], k[sl], v[sl], dout[sl], checkerboard, None)
    assert rel_err(dq[sl], rq) <= 5e-2 and rel_err(dk[sl], rk) <= 5e-2 and rel_err(dv[sl], rv) <= 5e-2
    a = (dq.double() * q.double()).sum(dim=(2, 3))
    b = (dk.double() * k.double()).sum(dim=(2, 3))
    assert ((a - b).abs() / (a.abs() + b.abs() + 1.0)).max().item() <= 5e-2
    out2, dq2, dk2, dv2 = _grads(q, k, v, dout, checkerboard, None)
    # dK and dV accumulate in a fixed order; dQ is summed over kv tiles by reduce-adds whose
    # order is not fixed, so it is reproducible only to fp32 summation noise
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    assert rel_err(dq2, dq) <= 1e-3
