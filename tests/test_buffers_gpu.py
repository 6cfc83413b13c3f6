"""GPU parity of mods that read captured buffers (the reference's score_mod_other_buffers /
mask_mod_other_buffers, flaxattention/core/attention.py:22-23, :35-52): a document mask over an
id tensor and a learned bias table, through create_block_mask, the forward, the backward and
the decode kernel, against the oracle evaluating the very same Python functions."""
import numpy as np
import pytest
import torch

from _util import DTYPES, lse_err, max_abs, normal, qkv, rel_err
from cases import TABLE_KEYS
from oracle.attention_oracle import attention_grads_oracle, flax_attention_oracle
from oracle.blockmask_oracle import create_block_mask_oracle

pytestmark = pytest.mark.gpu


def _documents(S, seed=7, device="cpu", dtype=torch.int64):
    """Document ids of a packed batch: non-decreasing, a few hundred tokens per document."""
    g = np.random.Generator(np.random.Philox(seed))
    cuts = np.sort(g.choice(np.arange(1, S), size=max(1, S // 200), replace=False))
    ids = np.searchsorted(cuts, np.arange(S), side="right")
    return torch.from_numpy(ids).to(dtype).to(device)


def _doc_causal(doc):
    def document_causal(b, h, q_idx, kv_idx):
        return (doc[q_idx] == doc[kv_idx]) & (q_idx >= kv_idx)

    return document_causal


def _bias_mod(table):
    def learned_bias(score, b, h, q_idx, kv_idx):
        return score + table[h, q_idx, kv_idx]

    return learned_bias


@pytest.mark.parametrize("where,dtype", [("cpu", torch.int64), ("cuda", torch.int32)])
def test_document_mask_tables_are_bit_exact(where, dtype):
    from flaxattention_b200 import create_block_mask

    S = 1024
    doc = _documents(S, device=where, dtype=dtype)
    bm = create_block_mask(_doc_causal(doc), 1, 1, S, S)
    torch.cuda.synchronize()
    want = create_block_mask_oracle(_doc_causal(doc.cpu()), 1, 1, S, S)
    for k in TABLE_KEYS:
        assert np.array_equal(getattr(bm, k).cpu().numpy(), want[k]), k
    assert 0 < bm.sparsity() < 100


@pytest.mark.parametrize("dt,D", [("f16", 64), ("bf16", 128), ("f32", 32)])
def test_document_mask_and_learned_bias_forward_backward(dt, D):
    """Both mods read a buffer; fp16 / D=64 runs the tcgen05 kernels, the others the general ones."""
    import flaxattention_b200 as fa

    B, H, S = 2, 2, 512
    doc = _documents(S)                                       # int64 on the CPU: copied to the GPU by the library
    table = 0.5 * normal(11, (H, S, S)).cuda()                # fp32 on the GPU: used in place
    mask, score = _doc_causal(doc), _bias_mod(table)
    q, k, v = qkv(B, H, H, S, S, D, dtype=DTYPES[dt])
    dout = normal(5, (B, H, S, D), DTYPES[dt])
    ref_out, ref_lse, rdq, rdk, rdv = attention_grads_oracle(q, k, v, dout, _bias_mod(table.cpu()), mask)
    fwd_out, fwd_lse = flax_attention_oracle(q, k, v, _bias_mod(table.cpu()), mask)

    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bm = fa.create_block_mask(mask, B, H, S, S)
    out, lse = fa.flax_attention(qc, kc, vc, score_mod=score, block_mask=bm, return_lse=True)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    tol = 1e-5 if dt == "f32" else 2e-2
    assert max_abs(out.detach().cpu(), fwd_out) <= tol * (10 if dt == "f32" else 1)
    err, same = lse_err(lse.detach().cpu(), fwd_lse)
    assert same and err <= tol * max(1.0, fwd_lse[torch.isfinite(fwd_lse)].abs().max().item()) * (10 if dt == "f32" else 1)
    gtol = 1e-4 if dt == "f32" else 5e-2
    for got, ref in ((qc.grad, rdq), (kc.grad, rdk), (vc.grad, rdv)):
        assert rel_err(got.cpu(), ref) <= gtol


def test_rebinding_the_same_source_to_other_tensors():
    """Two masks with identical generated code but different id tensors share a compiled module;
    each call must see its own tensor."""
    import flaxattention_b200 as fa

    S = 512
    q, k, v = qkv(1, 2, 2, S, S, 64, dtype=torch.float16)
    outs = []
    for seed in (3, 4, 3):
        doc = _documents(S, seed=seed)
        mask = _doc_causal(doc)
        bm = fa.create_block_mask(mask, 1, 2, S, S)
        out = fa.flax_attention(q.cuda(), k.cuda(), v.cuda(), block_mask=bm)
        torch.cuda.synchronize()
        ref, _ = flax_attention_oracle(q, k, v, None, mask)
        assert max_abs(out.cpu(), ref) <= 2e-2
        outs.append(out.cpu())
    assert max_abs(outs[0], outs[2]) == 0.0 and max_abs(outs[0], outs[1]) > 1e-3


def test_decode_with_a_document_mask():
    import flaxattention_b200 as fa

    B, H, Sq, Skv = 2, 4, 8, 2048
    doc_kv = _documents(Skv, seed=9)
    last = int(doc_kv[-1])

    def same_document_as_the_tail(b, h, q_idx, kv_idx):   # decode: the new tokens belong to the last document
        return doc_kv[kv_idx] == last

    q, k, v = qkv(B, H, H, Sq, Skv, 64, dtype=torch.float16)
    bm = fa.create_block_mask(same_document_as_the_tail, B, H, Sq, Skv)
    out, lse = fa.flax_attention(q.cuda(), k.cuda(), v.cuda(), block_mask=bm, return_lse=True,
                                 kernel_options={"path": "decode"})
    torch.cuda.synchronize()
    ref, ref_lse = flax_attention_oracle(q, k, v, None, same_document_as_the_tail)
    assert max_abs(out.cpu(), ref) <= 2e-2
    err, same = lse_err(lse.cpu(), ref_lse)
    assert same and err <= 2e-2 * max(1.0, ref_lse.abs().max().item())


def test_math_attention_with_explicit_other_buffers():
    """The reference's explicit form: mods that take the arrays as trailing arguments, passed in
    ``score_mod_other_buffers`` / ``mask_mod_other_buffers`` (core/attention.py:67-78)."""
    import math

    import flaxattention_b200 as fa

    B, H, S, D = 1, 2, 256, 64
    doc = _documents(S, device="cuda", dtype=torch.int32)
    table = normal(5, (H, S, S)).cuda()

    def score(s, b, h, q_idx, kv_idx, t):
        return s + t[h, q_idx, kv_idx]

    def mask(b, h, q_idx, kv_idx, ids):
        return (ids[q_idx] == ids[kv_idx]) & (q_idx >= kv_idx)

    q, k, v = qkv(B, H, H, S, S, D, dtype=torch.float16)
    bm = fa.create_block_mask(_doc_causal(doc), B, H, S, S)
    tup = bm.as_tuple()[:-1] + (mask,)
    out, lse2 = fa.math_attention(q.cuda(), k.cuda(), v.cuda(), score, tup, 0.125,
                                  score_mod_other_buffers=(table,), mask_mod_other_buffers=(doc,))
    torch.cuda.synchronize()
    ref, ref_lse = flax_attention_oracle(q, k, v, _bias_mod(table.cpu()), _doc_causal(doc.cpu()), 0.125)
    assert max_abs(out.cpu(), ref) <= 2e-2
    err, same = lse_err(lse2.cpu() * math.log(2.0), ref_lse)
    assert same and err <= 2e-2 * max(1.0, ref_lse.abs().max().item())


def test_compiled_block_mask_tables_are_kept():
    """create_block_mask(..., _compile=True) keeps the finished tables per (mask source, shape,
    block sizes, offsets, device): a repeated call returns the same tensors without a launch;
    masks over captured tensors are rebuilt every time."""
    from flaxattention_b200 import create_block_mask
    from flaxattention_b200.masks import causal_mask, generate_sliding_window

    a = create_block_mask(causal_mask, 2, 2, 512, 512, _compile=True)
    b = create_block_mask(causal_mask, 2, 2, 512, 512, _compile=True)
    assert b.kv_indices.data_ptr() == a.kv_indices.data_ptr() and b.q_num_blocks.data_ptr() == a.q_num_blocks.data_ptr()
    c = create_block_mask(causal_mask, 2, 2, 512, 512, _compile=True, h_offset=2)
    d = create_block_mask(generate_sliding_window(64), 2, 2, 512, 512, _compile=True)
    e = create_block_mask(causal_mask, 2, 2, 512, 512)
    assert len({t.kv_indices.data_ptr() for t in (a, c, d, e)}) == 4
    want = create_block_mask_oracle(causal_mask, 2, 2, 512, 512)
    for k in TABLE_KEYS:
        assert np.array_equal(getattr(b, k).cpu().numpy(), want[k]), k
    doc = _documents(512, device="cuda", dtype=torch.int32)
    m = _doc_causal(doc)
    f = create_block_mask(m, 1, 1, 512, 512, _compile=True)
    g = create_block_mask(m, 1, 1, 512, 512, _compile=True)
    assert f.kv_indices.data_ptr() != g.kv_indices.data_ptr()
