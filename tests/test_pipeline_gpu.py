"""HostPipeline (attention steps from pinned host buffers, copies overlapped with the kernels):
its results must equal those of one flax_attention_pallas call on the whole problem, on the
eager first pass, on the pass that records the CUDA graph and on replays with new data in the
same host buffers."""
import pytest
import torch

from _util import max_abs, normal, rel_err

pytestmark = pytest.mark.gpu


def _direct(fa, q, k, v, dout, score, bm, gqa):
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = fa.flax_attention_pallas(qc, kc, vc, score_mod=score, block_mask=bm, enable_gqa=gqa)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    return out.detach().cpu(), qc.grad.cpu(), kc.grad.cpu(), vc.grad.cpu()


@pytest.mark.parametrize("B,Hq,Hkv,S,D,chunks,dt", [
    (4, 4, 4, 512, 64, 8, torch.float16),     # more chunks than batch entries: heads are cut too
    (3, 8, 2, 384, 64, 2, torch.bfloat16),    # GQA, whole batch entries, a ragged last chunk
    (2, 8, 4, 256, 128, 16, torch.bfloat16),  # GQA cut in whole kv groups
])
def test_pipeline_equals_one_call(B, Hq, Hkv, S, D, chunks, dt):
    import flaxattention_b200 as fa
    from flaxattention_b200.masks import causal_mask
    from flaxattention_b200.mods import generate_alibi_bias

    alibi = generate_alibi_bias(Hq)
    bm = fa.create_block_mask(causal_mask, B, Hq, S, S)
    pipe = fa.HostPipeline(B, Hq, Hkv, S, S, D, dtype=dt, score_mod=alibi, block_mask=bm, chunks=chunks)
    assert pipe.use_graph and len(pipe.chunks) >= 2
    hq, hk, hv, hdo = (torch.empty(B, h, S, D, dtype=dt).pin_memory() for h in (Hq, Hkv, Hkv, Hq))
    ho, hdq, hdk, hdv = (torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv))
    for it in range(4):  # eager pass, graph capture, two replays
        for seed, t in ((10 * it + 1, hq), (10 * it, hk), (10 * it + 2, hv), (10 * it + 7, hdo)):
            t.copy_(normal(seed, tuple(t.shape), dt))
        pipe.step(hq, hk, hv, ho, hdq, hdk, hdv, hdout=hdo)
        torch.cuda.synchronize()
        fa.check_status()
        out, dq, dk, dv = _direct(fa, hq.clone(), hk.clone(), hv.clone(), hdo.clone(), alibi, bm, Hq != Hkv)
        assert torch.equal(ho, out), it
        assert torch.equal(hdk, dk) and torch.equal(hdv, dv), it
        assert rel_err(hdq, dq) <= 1e-3, it  # fp32 reduce-adds in an order that is not fixed
    assert len(pipe._graphs) == 1


def test_pipeline_forward_only_and_default_dout():
    import flaxattention_b200 as fa
    from flaxattention_b200.mods import checkerboard

    B, H, S, D = 4, 2, 256, 64
    q, k, v = (normal(s, (B, H, S, D), torch.float16).pin_memory() for s in (1, 0, 2))
    ho, hdq, hdk, hdv = (torch.empty_like(q).pin_memory() for _ in range(4))
    pipe = fa.HostPipeline(B, H, H, S, S, D, score_mod=checkerboard, chunks=4)
    for _ in range(3):
        pipe.step(q, k, v, ho, hdq, hdk, hdv)  # dO = 1
    torch.cuda.synchronize()
    out, dq, dk, dv = _direct(fa, q, k, v, torch.ones_like(q), checkerboard, None, False)
    assert torch.equal(ho, out) and torch.equal(hdk, dk) and torch.equal(hdv, dv) and rel_err(hdq, dq) <= 1e-3
    fwd = fa.HostPipeline(B, H, H, S, S, D, score_mod=checkerboard, chunks=2, backward=False)
    ho2 = torch.zeros_like(q).pin_memory()
    for _ in range(3):
        fwd.step(q, k, v, ho2)
    torch.cuda.synchronize()
    assert torch.equal(ho2, out)
    assert fwd.bytes_per_step() == (3 * q.numel() * 2, q.numel() * 2)


def test_pipeline_with_captured_tensors_runs_eagerly():
    """A mod that reads a tensor gets its address table refreshed before every launch, so these
    steps are not recorded into a graph; the results still equal a single call."""
    import flaxattention_b200 as fa

    B, H, S, D = 2, 2, 256, 64
    table = normal(5, (H, S, S)).cuda()

    def bias(score, b, h, q_idx, kv_idx):
        return score + table[h, q_idx, kv_idx]

    q, k, v = (normal(s, (B, H, S, D), torch.float16).pin_memory() for s in (1, 0, 2))
    ho, hdq, hdk, hdv = (torch.empty_like(q).pin_memory() for _ in range(4))
    pipe = fa.HostPipeline(B, H, H, S, S, D, score_mod=bias, chunks=2)
    assert not pipe.use_graph
    for _ in range(2):
        pipe.step(q, k, v, ho, hdq, hdk, hdv)
    torch.cuda.synchronize()
    out, dq, dk, dv = _direct(fa, q, k, v, torch.ones_like(q), bias, None, False)
    assert max_abs(ho, out) == 0.0 and torch.equal(hdk, dk) and torch.equal(hdv, dv) and rel_err(hdq, dq) <= 1e-3
