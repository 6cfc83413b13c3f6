"""Parity at the sizes of the benchmark configurations themselves.

The dense oracle cannot hold a whole configuration (the score tensor of B4 H16 S8192 is
17 GB), so each configuration runs at full size on the GPU and a slice of (batch, head)
pairs is compared with the oracle evaluated with the slice's global indices; the rest is
covered by properties that do not depend on the size: a batch x heads shard computed with
offsets equals the slice of the global result, and sum_q dQ.Q = sum_kv dK.K per head (both
equal sum(dS * S) for the bilinear score; an additive bias such as ALiBi does not change it).

Tolerances: O / LSE max-abs <= 2e-2 (LSE relative to its magnitude), gradients <= 5e-2
relative to the fp32 reference (the shape of the reference's own gradient checks,
tests/attention_test.py:385-477)."""
import pytest
import torch

from _util import lse_err, max_abs, normal, rel_err
from oracle.attention_oracle import attention_grads_oracle

pytestmark = pytest.mark.gpu


def _inputs(B, H, S, D, dtype):
    k = normal(0, (B, H, S, D), dtype)
    q = normal(1, (B, H, S, D), dtype)
    v = normal(2, (B, H, S, D), dtype)
    return q, k, v


def _compare_slice(sl, b0, h0, host, dev, dout_host, score, mask):
    q, k, v = host
    out, lse, dq, dk, dv = dev
    r_out, r_lse, rq, rk, rv = attention_grads_oracle(q[sl], k[sl], v[sl], dout_host[sl], score, mask,
                                                      b_offset=b0, h_offset=h0)
    assert max_abs(out[sl].cpu(), r_out) <= 2e-2
    err, same = lse_err(lse[sl].cpu(), r_lse)
    assert same and err <= 2e-2 * max(1.0, r_lse[torch.isfinite(r_lse)].abs().max().item())
    for name, g, r in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        assert rel_err(g[sl].cpu(), r) <= 5e-2, f"{name}: {rel_err(g[sl].cpu(), r)}"


def _run(fa, q, k, v, dout, score, bm, **kw):
    qc, kc, vc = (t.detach().requires_grad_(True) for t in (q, k, v))
    out, lse = fa.flax_attention_pallas(qc, kc, vc, score_mod=score, block_mask=bm, return_lse=True, **kw)
    out.backward(dout)
    return out.detach(), lse, qc.grad, kc.grad, vc.grad


def test_causal_alibi_configuration_at_full_size():
    """B8 H8 S2048 D64 bf16, causal BlockMask (block 128) + ALiBi, forward and gradients."""
    import flaxattention_b200 as fa
    from flaxattention_b200.masks import causal_mask
    from flaxattention_b200.mods import generate_alibi_bias

    B, H, S, D = 8, 8, 2048, 64
    alibi = generate_alibi_bias(H)
    host = _inputs(B, H, S, D, torch.bfloat16)
    dout_h = normal(7, (B, H, S, D), torch.bfloat16)
    q, k, v = (t.cuda() for t in host)
    dout = dout_h.cuda()
    bm = fa.create_block_mask(causal_mask, B, H, S, S)
    assert abs(bm.sparsity() - 46.875) < 1e-3
    dev = _run(fa, q, k, v, dout, alibi, bm)
    torch.cuda.synchronize()
    fa.check_status()
    # the steepest and the flattest ALiBi slope
    _compare_slice((slice(0, 1), slice(0, 1)), 0, 0, host, dev, dout_h, alibi, causal_mask)
    _compare_slice((slice(7, 8), slice(7, 8)), 7, 7, host, dev, dout_h, alibi, causal_mask)
    out, lse, dq, dk, dv = dev
    # both sums cancel heavily with a random dO, so the difference is measured against the sums of
    # absolute values
    a = (dq.double() * q.double()).sum(dim=(2, 3))
    b = (dk.double() * k.double()).sum(dim=(2, 3))
    den = (dq.double() * q.double()).abs().sum(dim=(2, 3)) + (dk.double() * k.double()).abs().sum(dim=(2, 3))
    assert ((a - b).abs() / den).max().item() <= 1e-2
    # shard (b 4..7, h 2..5) with global offsets
    sl = (slice(4, 8), slice(2, 6))
    part = _run(fa, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), dout[sl].contiguous(), alibi,
                bm.shard(*sl), b_offset=4, h_offset=2)
    torch.cuda.synchronize()
    assert torch.equal(part[0], out[sl]) and torch.equal(part[1], lse[sl])
    assert torch.equal(part[3], dk[sl]) and torch.equal(part[4], dv[sl])
    assert rel_err(part[2], dq[sl]) <= 1e-3  # dQ is summed by reduce-adds whose order is not fixed


def test_attention_sink_configuration_at_full_size():
    """B4 H16 S8192 D128 bf16, generate_attention_sink(1024, 4) BlockMask (block 128):
    85.5 % of the blocks are skipped.  One (batch, head) pair against the oracle, and the 4 x 2
    batch x heads partition of this configuration (shard b = 3, heads 8..15) against the global run."""
    import flaxattention_b200 as fa
    from flaxattention_b200.masks import generate_attention_sink

    B, H, S, D = 4, 16, 8192, 128
    sink = generate_attention_sink(1024, 4)
    host = _inputs(B, H, S, D, torch.bfloat16)
    dout_h = normal(7, (B, H, S, D), torch.bfloat16)
    q, k, v = (t.cuda() for t in host)
    dout = dout_h.cuda()
    bm = fa.create_block_mask(sink, B, H, S, S)
    assert abs(bm.sparsity() - 100.0 * 3501 / 4096) < 1e-3
    dev = _run(fa, q, k, v, dout, None, bm)
    torch.cuda.synchronize()
    fa.check_status()
    _compare_slice((slice(2, 3), slice(9, 10)), 2, 9, host, dev, dout_h, None, sink)
    out, lse, dq, dk, dv = dev
    sl = (slice(3, 4), slice(8, 16))
    part = _run(fa, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), dout[sl].contiguous(), None,
                bm.shard(*sl), b_offset=3, h_offset=8)
    torch.cuda.synchronize()
    assert torch.equal(part[0], out[sl]) and torch.equal(part[1], lse[sl])
    assert rel_err(part[2], dq[sl]) <= 1e-3 and rel_err(part[3], dk[sl]) <= 1e-3 and rel_err(part[4], dv[sl]) <= 1e-3


def test_head_dependent_mods_see_global_indices_in_a_shard():
    """A mask and a bias that depend on b and h: a shard with non-zero b_offset and h_offset
    must reproduce the slice of the global result (forward and gradients)."""
    import flaxattention_b200 as fa
    from cases import head_dependent
    from flaxattention_b200.mods import generate_alibi_bias

    B, H, S, D = 4, 8, 512, 128
    alibi = generate_alibi_bias(H)
    host = _inputs(B, H, S, D, torch.float16)
    q, k, v = (t.cuda() for t in host)
    dout = normal(7, (B, H, S, D), torch.float16).cuda()
    bm = fa.create_block_mask(head_dependent, B, H, S, S)
    full = _run(fa, q, k, v, dout, alibi, bm)
    sl = (slice(1, 3), slice(4, 8))
    bm_shard = fa.create_block_mask(head_dependent, 2, 4, S, S, b_offset=1, h_offset=4)
    for key in ("kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices"):
        assert torch.equal(getattr(bm_shard, key), getattr(bm, key)[sl]), key
    part = _run(fa, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), dout[sl].contiguous(), alibi,
                bm_shard, b_offset=1, h_offset=4)
    torch.cuda.synchronize()
    fa.check_status()
    assert torch.equal(part[0], full[0][sl]) and torch.equal(part[1], full[1][sl])
    for i in (2, 3, 4):
        assert rel_err(part[i], full[i][sl]) <= 1e-3
