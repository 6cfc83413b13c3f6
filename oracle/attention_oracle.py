"""Dense CPU restatement of the reference's pure-JAX attention.  TEST INFRASTRUCTURE ONLY.

Follows, operation by operation:
  flax_attention           flaxattention/core/attention.py:169-218   (defaults, LSE units)
  math_attention           flaxattention/core/attention.py:67-106    (GQA repeat, logsumexp,
                                                                      masked-row fix, softmax, P.V)
  _math_attention_inner    flaxattention/core/attention.py:14-65     (Q.K^T in the input dtype,
                                                                      scale, vmapped mods, where(mask))
  _vmap_for_bhqkv          flaxattention/core/common.py:41-81        (index semantics: int32 aranges)

Pinning: JAX is not installed where this file was written, so the reference itself could
not be run.  The restatement is pinned against eager torch ``flex_attention`` on CPU, the
oracle the reference's own tests use (tests/attention_test.py:14-63, decimal=2), through the
fixtures in tests/golden/ (made by tests/golden/make_golden.py).  Gradients, fp16/bf16 and
real masks are not covered by any stored vector of the reference: for those, parity is
unpinned by the reference and defined by this restatement of its source.

The mods are ordinary Python callables; they are called once with broadcast int32 index
tensors ``b[B,1,1,1], h[1,H,1,1], q[1,1,Sq,1], kv[1,1,1,Skv]``, which is what the four
nested vmaps of the reference amount to.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch


def _indices(B, H, Sq, Skv, b_offset=0, h_offset=0):
    b = (torch.arange(B, dtype=torch.int32) + b_offset).view(B, 1, 1, 1)
    h = (torch.arange(H, dtype=torch.int32) + h_offset).view(1, H, 1, 1)
    q = torch.arange(Sq, dtype=torch.int32).view(1, 1, Sq, 1)
    kv = torch.arange(Skv, dtype=torch.int32).view(1, 1, 1, Skv)
    return b, h, q, kv


def dense_mask(mask_mod: Optional[Callable], B, H, Sq, Skv, b_offset=0, h_offset=0) -> torch.Tensor:
    """Boolean [B,H,Sq,Skv] mask (True = keep)."""
    if mask_mod is None:
        return torch.ones(B, H, Sq, Skv, dtype=torch.bool)
    b, h, q, kv = _indices(B, H, Sq, Skv, b_offset, h_offset)
    m = mask_mod(b, h, q, kv)
    if not isinstance(m, torch.Tensor):
        m = torch.as_tensor(m)
    return m.to(torch.bool).expand(B, H, Sq, Skv)


def post_mod_scores(query, key, score_mod, mask_mod, scale, *, matmul_in_input_dtype=True,
                    work_dtype=torch.float32, b_offset=0, h_offset=0) -> torch.Tensor:
    """_math_attention_inner: scores after scale, score_mod and mask (masked = -inf).
    query [B,H,Sq,D], key [B,H,Skv,D] (kv heads already repeated)."""
    B, H, Sq, _ = query.shape
    Skv = key.shape[2]
    if matmul_in_input_dtype:
        scores = torch.matmul(query, key.transpose(-2, -1)).to(work_dtype)
    else:
        scores = torch.matmul(query.to(work_dtype), key.to(work_dtype).transpose(-2, -1))
    scores = scores * scale
    b, h, q, kv = _indices(B, H, Sq, Skv, b_offset, h_offset)
    if score_mod is not None:
        scores = score_mod(scores, b, h, q, kv)
        if scores.dtype != work_dtype:
            scores = scores.to(work_dtype)
    mask = dense_mask(mask_mod, B, H, Sq, Skv, b_offset, h_offset)
    return torch.where(mask, scores, torch.full((), -math.inf, dtype=work_dtype))


def flax_attention_oracle(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                          score_mod: Optional[Callable] = None, mask_mod: Optional[Callable] = None,
                          scale: Optional[float] = None, *, matmul_in_input_dtype: bool = True,
                          work_dtype=torch.float32, b_offset: int = 0, h_offset: int = 0
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (output [B,Hq,Sq,Dv] in the input dtype, natural-log LSE [B,Hq,Sq] in
    ``work_dtype``).  Differentiable with torch autograd.  Fully masked rows give output 0
    and LSE -inf (core/attention.py:97-104).

    ``matmul_in_input_dtype=True`` reproduces the reference exactly (Q.K^T and P.V are
    computed in the input dtype); ``False`` with ``work_dtype=float32/float64`` is the
    high-precision reference used for gradient tolerances."""
    B, Hq, Sq, D = query.shape
    Hkv = key.shape[1]
    G = Hq // Hkv
    if G > 1:
        key = key.repeat_interleave(G, dim=1)
        value = value.repeat_interleave(G, dim=1)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    s = post_mod_scores(query, key, score_mod, mask_mod, scale, matmul_in_input_dtype=matmul_in_input_dtype,
                        work_dtype=work_dtype, b_offset=b_offset, h_offset=h_offset)
    masked_rows = torch.all(s == -math.inf, dim=-1)
    safe = torch.where(masked_rows[..., None], torch.zeros((), dtype=work_dtype), s)
    lse = torch.logsumexp(safe, dim=-1)
    lse = torch.where(masked_rows, torch.full((), -math.inf, dtype=work_dtype), lse)
    p = torch.softmax(safe, dim=-1)
    p = torch.where(masked_rows[..., None], torch.zeros((), dtype=work_dtype), p)
    if matmul_in_input_dtype:
        out = torch.matmul(p.to(query.dtype), value)
    else:
        out = torch.matmul(p, value.to(work_dtype)).to(query.dtype)
    return out, lse


def flax_attention_oracle_chunked(query, key, value, score_mod=None, mask_mod=None, scale=None, *,
                                  chunk_bh: int = 8, **kw):
    """Forward only, evaluated in chunks of heads so that the [B,H,Sq,Skv] score tensor of
    a large problem never exists at once."""
    B, Hq, Sq, D = query.shape
    Hkv = key.shape[1]
    G = Hq // Hkv
    outs, lses = [], []
    with torch.no_grad():
        for b in range(B):
            ob, lb = [], []
            for h0 in range(0, Hq, chunk_bh):
                h1 = min(Hq, h0 + chunk_bh)
                kh = key[b:b + 1, h0 // G:(h1 - 1) // G + 1]
                vh = value[b:b + 1, h0 // G:(h1 - 1) // G + 1]
                if G > 1:
                    kh = kh.repeat_interleave(G, dim=1)[:, h0 % G:h0 % G + (h1 - h0)]
                    vh = vh.repeat_interleave(G, dim=1)[:, h0 % G:h0 % G + (h1 - h0)]
                o, l = flax_attention_oracle(query[b:b + 1, h0:h1], kh, vh, score_mod, mask_mod, scale,
                                             b_offset=kw.get("b_offset", 0) + b,
                                             h_offset=kw.get("h_offset", 0) + h0,
                                             matmul_in_input_dtype=kw.get("matmul_in_input_dtype", True),
                                             work_dtype=kw.get("work_dtype", torch.float32))
                ob.append(o)
                lb.append(l)
            outs.append(torch.cat(ob, dim=1))
            lses.append(torch.cat(lb, dim=1))
    return torch.cat(outs, dim=0), torch.cat(lses, dim=0)


def attention_grads_oracle(query, key, value, dout, score_mod=None, mask_mod=None, scale=None, *,
                           work_dtype=torch.float32, b_offset=0, h_offset=0):
    """(out, lse, dq, dk, dv) of the high-precision reference: inputs are upcast to
    ``work_dtype`` and differentiated with autograd."""
    q = query.detach().to(work_dtype).requires_grad_(True)
    k = key.detach().to(work_dtype).requires_grad_(True)
    v = value.detach().to(work_dtype).requires_grad_(True)
    out, lse = flax_attention_oracle(q, k, v, score_mod, mask_mod, scale, matmul_in_input_dtype=False,
                                     work_dtype=work_dtype, b_offset=b_offset, h_offset=h_offset)
    out.backward(dout.to(work_dtype))
    return out.detach(), lse.detach(), q.grad, k.grad, v.grad
