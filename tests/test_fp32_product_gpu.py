"""GPU parity of the kernel variants that keep the fp32 Q.K^T product (compiled without the
rounding of the scores to the input dtype): what ``flax_attention_pallas`` runs, what
``kernel_options={"round_scores": False}`` selects, and what bench.py times.

The reference's fused kernel keeps the fp32 product (flaxattention/kernel/attention.py:82),
so the oracle is used in its ``matmul_in_input_dtype=False`` mode.  Shapes are ones the
tcgen05 kernels cover (fp16 / bf16, head dim 64 or 128, at least 128 rows); in these variants
the forward without a score_mod leaves the raw scores untouched and folds the scale into the
exponent, takes every fourth pair of exponentials as a polynomial, and the backward works on
packed fp32 pairs when the score_mod is affine or absent.

Tolerances: O and LSE max-abs <= 2e-2; gradients <= 5e-2 relative to the fp32 reference."""
import math

import numpy as np
import pytest
import torch

from _util import DTYPES, lse_err, max_abs, normal, qkv, rel_err
from oracle.attention_oracle import attention_grads_oracle

pytestmark = pytest.mark.gpu


def _mods(score, mask, Hq):
    from flaxattention_b200 import fnp
    from flaxattention_b200.masks import causal_mask, generate_attention_sink, generate_sliding_window
    from flaxattention_b200.mods import checkerboard, generate_alibi_bias

    def softcap(s, b, h, q, kv):
        return 20.0 * fnp.tanh(s / 20.0)

    def relbias(s, b, h, q, kv):
        # multiplier without indices, bias linear in q and in kv with a slope per (batch, head): the kernels
        # take the bias once per chunk and add multiples of the slope
        return s * 1.5 + fnp.float32(kv - 2 * q) * (0.002 * fnp.float32(h + 1 + b))

    def halfbias(s, b, h, q, kv):
        # linear in kv only (the bias is quadratic in q): the forward uses the slope, the backward does not
        return s + fnp.float32(q) * fnp.float32(q) * 1e-5 - 0.01 * fnp.float32(kv)

    s = {None: None, "alibi": generate_alibi_bias(Hq), "checker": checkerboard, "softcap": softcap,
         "relbias": relbias, "halfbias": halfbias}[score]
    m = {None: None, "causal": causal_mask, "sink": generate_attention_sink(200, 4),
         "window": generate_sliding_window(100)}[mask]
    return s, m


def _check_all(got, ref, dt="f16"):
    out, lse, dq, dk, dv = got
    r_out, r_lse, rq, rk, rv = ref
    assert not torch.isnan(out.float()).any()
    assert max_abs(out, r_out) <= 2e-2
    err, same = lse_err(lse, r_lse)
    fin = torch.isfinite(r_lse)
    assert same and err <= 2e-2 * (max(1.0, r_lse[fin].abs().max().item()) if fin.any() else 1.0)
    for name, g, r in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        assert not torch.isnan(g.float()).any(), name
        assert rel_err(g, r) <= 5e-2, f"{name}: {rel_err(g, r)}"


CASES = [
    # B, Hq, Hkv, Sq, Skv, D, dtype, score, mask, tables
    (1, 2, 2, 256, 256, 64, "f16", None, None, False),        # raw scores + polynomial exponentials
    (1, 2, 2, 384, 512, 64, "bf16", None, None, False),
    (2, 2, 2, 512, 512, 64, "f16", "checker", None, False),   # affine: packed fp32 pairs in the backward
    (1, 4, 4, 512, 512, 64, "bf16", "alibi", "causal", True),
    (1, 4, 2, 512, 768, 64, "f16", "softcap", "window", True),  # not affine: scalar path with the derivative
    (1, 2, 2, 300, 333, 64, "f16", "alibi", "causal", True),  # ragged
    (1, 2, 2, 512, 512, 64, "f16", None, "causal", False),    # mask_mod on every tile, no tables
    (1, 2, 2, 512, 512, 128, "bf16", None, "sink", True),
    (1, 2, 2, 256, 640, 128, "f16", "checker", None, False),
    (1, 2, 2, 384, 384, 128, "bf16", "alibi", "causal", False),
    (2, 2, 2, 384, 512, 64, "bf16", "relbias", "causal", True),   # index-linear bias: slope path in both kernels
    (1, 2, 2, 256, 384, 128, "f16", "relbias", None, False),
    (1, 2, 2, 384, 384, 64, "f16", "halfbias", "window", True),   # linear in kv only
]


@pytest.mark.parametrize("entry", ["pallas", "flax_option"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_fp32_product_variants_match_the_reference(case, entry):
    import flaxattention_b200 as fa

    B, Hq, Hkv, Sq, Skv, D, dt, score, mask, tables = case
    s, m = _mods(score, mask, Hq)
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, dtype=DTYPES[dt])
    dout = normal(7, (B, Hq, Sq, D), DTYPES[dt])
    ref = attention_grads_oracle(q, k, v, dout, s, m)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bm = None
    if m is not None:
        if tables:
            bm = fa.create_block_mask(m, B, Hq, Sq, Skv)
        elif entry == "flax_option":
            bm = fa.blockmask._create_empty_block_mask(qc, kc)
            bm.mask_mod = m
    if entry == "pallas":
        out, lse = fa.flax_attention_pallas(qc, kc, vc, score_mod=s, mask_mod=m, block_mask=bm, enable_gqa=Hq != Hkv,
                                            return_lse=True)
    else:
        out, lse = fa.flax_attention(qc, kc, vc, score_mod=s, block_mask=bm, enable_gqa=Hq != Hkv, return_lse=True,
                                     kernel_options={"round_scores": False, "path": "fwd"})
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    fa.check_status()
    _check_all((out.detach().cpu(), lse.cpu(), qc.grad.cpu(), kc.grad.cpu(), vc.grad.cpu()), ref, dt)


@pytest.mark.parametrize("D", [64, 128])
def test_sequence_major_layout_on_the_tcgen05_kernels(D):
    """bhln=False ([B, L, H, N]): the TMA tensor maps then have the head stride below the row
    stride, and dQ / dK / dV are written through the same strides."""
    import flaxattention_b200 as fa
    from flaxattention_b200.masks import causal_mask
    from flaxattention_b200.mods import generate_alibi_bias

    B, H, S = 2, 4, 384
    alibi = generate_alibi_bias(H)
    q, k, v = qkv(B, H, H, S, S, D, dtype=torch.bfloat16)
    dout = normal(7, (B, H, S, D), torch.bfloat16)
    ref = attention_grads_oracle(q, k, v, dout, alibi, causal_mask)
    qc, kc, vc = (t.transpose(1, 2).contiguous().cuda().requires_grad_(True) for t in (q, k, v))
    bm = fa.create_block_mask(causal_mask, B, H, S, S)
    out, lse = fa.flax_attention_pallas(qc, kc, vc, score_mod=alibi, block_mask=bm, bhln=False, return_lse=True)
    assert out.shape == (B, S, H, D)
    out.backward(dout.transpose(1, 2).contiguous().cuda())
    torch.cuda.synchronize()
    fa.check_status()
    back = lambda t: t.detach().cpu().transpose(1, 2)  # noqa: E731
    _check_all((back(out), lse.cpu(), back(qc.grad), back(kc.grad), back(vc.grad)), ref)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_rows_without_a_visible_key_inside_a_visited_tile(dt):
    """mask = kv + 10 <= q: rows 0-9 see no key, but their tile is visited because the other
    rows of the block do.  Output exactly 0 and LSE -inf, also in the variant that takes part
    of the exponentials as a polynomial (which returns a tiny positive number for -inf)."""
    import flaxattention_b200 as fa

    def shifted(b, h, q, kv):
        return kv + 10 <= q

    q, k, v = (t.cuda() for t in qkv(1, 2, 2, 256, 256, 64, dtype=DTYPES[dt]))
    bm = fa.create_block_mask(shifted, 1, 2, 256, 256)
    o1, l1 = fa.flax_attention(q, k, v, block_mask=bm, return_lse=True)
    o2, l2 = fa.flax_attention_pallas(q, k, v, mask_mod=shifted, return_lse=True)
    o3, l3 = fa.flax_attention_pallas(q, k, v, block_mask=bm, return_lse=True)
    torch.cuda.synchronize()
    for o, l in ((o1, l1), (o2, l2), (o3, l3)):
        assert torch.count_nonzero(o[:, :, :10]) == 0
        assert bool(torch.isneginf(l[:, :, :10]).all())
        assert bool(torch.isfinite(l[:, :, 10:]).all()) and not torch.isnan(o.float()).any()


def test_benchmark_call_matches_the_reference():
    """The exact call bench.py times: B8 H8 S2048 D64 fp16, checkerboard, no mask, scores kept
    in fp32, through ``attention._Call`` / ``_forward`` / ``_backward``; one batch entry and two
    heads are compared with the reference."""
    from flaxattention_b200 import attention as A
    from flaxattention_b200.mods import checkerboard

    B, H, S, D = 8, 8, 2048, 64
    q, k, v = qkv(B, H, H, S, S, D, dtype=torch.float16)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    dout = torch.ones(B, H, S, D, dtype=torch.float16, device="cuda")
    call = A._Call(qc, kc, vc, checkerboard, None, None, 1.0 / math.sqrt(D), "bhsd", 0, 0, {"flags": 0})
    out, lse = A._forward(call, qc, kc, vc)
    dq, dk, dv = A._backward(call, qc, kc, vc, out, lse, dout)
    torch.cuda.synchronize()
    A.check_status()
    sl = (slice(5, 6), slice(3, 5))
    ref = attention_grads_oracle(q[sl], k[sl], v[sl], dout[sl].cpu(), checkerboard, None, b_offset=5, h_offset=3)
    _check_all((out[sl].cpu(), lse[sl].cpu(), dq[sl].cpu(), dk[sl].cpu(), dv[sl].cpu()), ref)
    # and without a score_mod: the forward path that never rewrites the scores
    call0 = A._Call(qc, kc, vc, A._identity, None, None, 1.0 / math.sqrt(D), "bhsd", 0, 0, {"flags": 0})
    out0, lse0 = A._forward(call0, qc, kc, vc)
    dq0, dk0, dv0 = A._backward(call0, qc, kc, vc, out0, lse0, dout)
    torch.cuda.synchronize()
    A.check_status()
    ref0 = attention_grads_oracle(q[sl], k[sl], v[sl], dout[sl].cpu())
    _check_all((out0[sl].cpu(), lse0[sl].cpu(), dq0[sl].cpu(), dk0[sl].cpu(), dv0[sl].cpu()), ref0)


def test_profile_times_cover_every_kernel_of_a_call():
    """fa_profile_enable / fa_profile_read: names and device times of the kernels of the most
    recent call, results unchanged."""
    from flaxattention_b200 import _cabi
    from flaxattention_b200 import attention as A

    q, k, v = (t.cuda() for t in qkv(1, 2, 2, 512, 512, 64, dtype=torch.float16))
    dout = torch.ones_like(q)
    call = A._Call(q, k, v, A._identity, None, None, 0.125, "bhsd", 0, 0, None)
    out, lse = A._forward(call, q, k, v)
    want = A._backward(call, q, k, v, out, lse, dout)
    _cabi.profile_enable(True)
    try:
        A._forward(call, q, k, v)
        fwd = _cabi.profile_read()
        got = A._backward(call, q, k, v, out, lse, dout)
        bwd = _cabi.profile_read()
    finally:
        _cabi.profile_enable(False)
    assert [n for n, _ in fwd] == ["fa_fwd_tc_kernel"]
    assert [n for n, _ in bwd] == ["fa_bwd_prep_kernel", "fa_bwd_tc_kernel", "fa_dq_convert_kernel"]
    assert all(0.0 < ms < 50.0 for _, ms in fwd + bwd)
    assert torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])
    assert np.isfinite(got[0].float().cpu().numpy()).all()
