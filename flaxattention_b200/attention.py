"""Public attention entry points, same names and arguments as the reference
(flaxattention/core/attention.py): ``flax_attention`` (:169-218), ``flax_attention_pallas``
(:220-312) and ``math_attention`` (:67-106).

All three run the hand-written sm_100a kernels through the C ABI (``_cabi``): the flash
forward (or the split-KV decode kernel for short query blocks), and the flash backward
through ``torch.autograd`` where the reference uses ``jax.custom_vjp``
(flaxattention/kernel/attention.py:166-168, :653).  Inputs are torch CUDA tensors; numpy
arrays are copied to the current CUDA device and the result is copied back.  There is no
CPU implementation.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Optional, Tuple, Union

import numpy as np
import torch

from . import _cabi
from .blockmask import BlockMask, bind_mod_buffers, module_for, noop_mask

_DTYPES = {torch.float16: _cabi.FA_F16, torch.bfloat16: _cabi.FA_BF16, torch.float32: _cabi.FA_F32}

# decode path: query blocks of at most this many rows go through the split-KV kernel
DECODE_MAX_SQ = 64
DECODE_MIN_SKV = 512


def _identity(score, batch, head, token_q, token_kv):
    return score


def _validate_sdpa_input(query, key, value):
    if query.dtype != key.dtype or query.dtype != value.dtype:
        raise ValueError(
            f"Expected query, key, and value to have the same dtype, "
            f"but got query.dtype: {query.dtype}, key.dtype: {key.dtype}, "
            f"and value.dtype: {value.dtype} instead."
        )
    if query.ndim < 2 or key.ndim < 2 or value.ndim < 2:
        raise ValueError(
            f"Expected query, key, and value to all be  at least 2 dimensional, but got query.dim: "
            f"{query.ndim}, key.dim: {key.ndim} and value.dim: {value.ndim} instead."
        )


def _validate_embed_dim(query, key, value):
    if query.shape[-1] != key.shape[-1]:
        raise ValueError(
            f"Expect query and key/value to have the same embedding dimension "
            f"but got E={query.shape[-1]} and E={key.shape[-1]}."
        )
    if value.shape[-1] > query.shape[-1]:
        raise ValueError(
            f"NYI: Currently value embedding dimension must be less than or equal to query embedding dimension. "
            f"Got Ev={value.shape[-1]} and E={query.shape[-1]}."
        )


def _validate_heads(hq: int, hkv: int, enable_gqa: bool):
    if (not enable_gqa) and hq != hkv:
        raise ValueError(
            f"Expect query and key/value to have the same number of heads "
            f"but got Hq={hq} and Hkv={hkv}. "
            f"Try setting enable_gqa=True for GQA."
        )
    if enable_gqa and hq % hkv != 0:
        raise ValueError(
            f"Expect number of query heads to be a multiple of kv heads for GQA "
            f"but got Hq={hq} and Hkv={hkv}."
        )


# --------------------------------------------------------------------------------------
# C-ABI call plumbing
# --------------------------------------------------------------------------------------
# One status word for the whole process, in pinned host memory (which every GPU can address):
# the tcgen05 kernels OR FA_STATUS_WAIT_TIMEOUT into it when one of their bounded barrier waits
# runs out, and the host can look at it at any time without synchronising.  It is checked at
# the start of the next call and by ``check_status()``.
_status_word: Optional[torch.Tensor] = None


def _status() -> torch.Tensor:
    global _status_word
    if _status_word is None:
        _status_word = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _status_word


def check_status() -> None:
    """Raises ``FlaxAttnError`` if a kernel launched earlier through this module reported an
    error (a barrier wait that ran out: the results of that launch are incomplete).  Call it
    after synchronising to be sure about the launches issued so far; every attention call also
    runs it first, so an error surfaces at the latest on the next call."""
    w = _status_word
    if w is not None and int(w[0]) != 0:
        bits = int(w[0])
        w[0] = 0
        raise _cabi.FlaxAttnError(-3, f"a kernel reported status bits {bits:#x} (bit 0: a bounded barrier wait ran out; "
                                      "bit 1: a launch configuration the kernel refused); the results of that launch "
                                      "are incomplete")


def _tensor(t: torch.Tensor, layout: str) -> _cabi.FaTensor:
    """layout 'bhsd' or 'bshd'; the last dim must be contiguous."""
    if t.stride(-1) != 1:
        raise ValueError("the head dimension must be contiguous")
    if layout == "bhsd":
        return _cabi.FaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return _cabi.FaTensor(t.data_ptr(), t.stride(0), t.stride(2), t.stride(1))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class _Call:
    """Everything one attention problem needs besides q/k/v: shapes, mods, tables."""

    def __init__(self, query, key, value, score_mod, mask_mod, block_mask: Optional[BlockMask], scale, layout,
                 b_offset, h_offset, options, round_scores=False):
        if query.device.type != "cuda":
            raise RuntimeError("flaxattention_b200 runs on CUDA tensors only; there is no CPU path")
        if query.dtype not in _DTYPES:
            raise ValueError(f"unsupported dtype {query.dtype}; use float16, bfloat16 or float32")
        self.layout = layout
        if layout == "bhsd":
            self.B, self.Hq, self.Sq, self.D = query.shape
            _, self.Hkv, self.Skv, self.Dv = value.shape
        else:
            self.B, self.Sq, self.Hq, self.D = query.shape
            _, self.Skv, self.Hkv, self.Dv = value.shape
        self.dtype = query.dtype
        self.scale = float(scale)
        self.b_offset, self.h_offset = int(b_offset), int(h_offset)
        self.block_mask = block_mask
        if block_mask is not None and block_mask.kv_indices.ndim != 4:
            raise ValueError("BlockMask tables must be 4-dimensional [B, H, nQ, nKV]")
        self.module = module_for(score_mod, mask_mod)
        self.score_mod, self.mask_mod = score_mod, mask_mod
        self.options = dict(options or {})
        self.round_scores = bool(self.options.get("round_scores", round_scores))

    def params(self, q, k, v, o, lse) -> _cabi.FaAttnParams:
        p = _cabi.FaAttnParams()
        p.dtype = _DTYPES[self.dtype]
        p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.D, p.Dv = self.B, self.Hq, self.Hkv, self.Sq, self.Skv, self.D, self.Dv
        p.scale = self.scale
        p.b_offset, p.h_offset = self.b_offset, self.h_offset
        p.q, p.k, p.v, p.o = (_tensor(t, self.layout) for t in (q, k, v, o))
        p.lse = _ptr(lse)
        p.flags = (_cabi.FLAG_ROUND_SCORES if self.round_scores else 0) | int(self.options.get("flags", 0))
        if self.options.get("kernels") == "general":
            p.flags |= _cabi.FLAG_GENERAL_KERNELS
        st = self.options.get("status")  # optional int32 CUDA tensor the kernels OR error bits into
        p.status = (st if st is not None else _status()).data_ptr()
        bm = self.block_mask
        if bm is not None:
            t = p.tables
            if bm.kv_num_blocks.device != q.device:
                raise ValueError("the BlockMask tables live on a different device than the inputs")
            t.kv_num_blocks, t.kv_indices = _ptr(bm.kv_num_blocks), _ptr(bm.kv_indices)
            t.full_kv_num_blocks, t.full_kv_indices = _ptr(bm.full_kv_num_blocks), _ptr(bm.full_kv_indices)
            t.q_num_blocks, t.q_indices = _ptr(bm.q_num_blocks), _ptr(bm.q_indices)
            t.full_q_num_blocks, t.full_q_indices = _ptr(bm.full_q_num_blocks), _ptr(bm.full_q_indices)
            t.mask_B, t.mask_H = bm.kv_indices.shape[0], bm.kv_indices.shape[1]
            t.num_q_blocks, t.num_kv_blocks = bm.kv_indices.shape[2], bm.kv_indices.shape[3]
            t.q_block_size, t.kv_block_size = bm.BLOCK_SIZE
            mb = getattr(bm, "mask_bits", None)
            if mb is not None and self.mask_mod is bm.mask_mod and mb.device == q.device and mb.shape[2] >= self.Sq \
                    and mb.shape[3] * 32 >= self.Skv and mb.shape[0] in (1, self.B) and mb.shape[1] in (1, self.Hq):
                if mb.dtype != torch.int32 or not mb.is_contiguous():
                    raise ValueError("BlockMask.mask_bits must be a contiguous int32 tensor")
                t.mask_bits, t.mask_bits_stride, t.mask_bits_rows = mb.data_ptr(), mb.shape[3], mb.shape[2]
                t.mask_bits_B, t.mask_bits_H = mb.shape[0], mb.shape[1]
            for x in (bm.kv_num_blocks, bm.kv_indices, bm.full_kv_num_blocks, bm.full_kv_indices, bm.q_num_blocks,
                      bm.q_indices, bm.full_q_num_blocks, bm.full_q_indices):
                if x is not None and (x.dtype != torch.int32 or not x.is_contiguous()):
                    raise ValueError("BlockMask tables must be contiguous int32 tensors")
        return p

    def use_decode(self) -> bool:
        force = self.options.get("path")
        if force == "decode":
            return True
        if force == "fwd":
            return False
        return self.Sq <= DECODE_MAX_SQ and self.Skv >= DECODE_MIN_SKV and self.dtype != torch.float32

    def out_like(self, query):
        if self.layout == "bhsd":
            return torch.empty(self.B, self.Hq, self.Sq, self.Dv, dtype=query.dtype, device=query.device)
        return torch.empty(self.B, self.Sq, self.Hq, self.Dv, dtype=query.dtype, device=query.device)


def _forward(call: _Call, q, k, v):
    L = _cabi.lib()
    check_status()
    out = call.out_like(q)
    lse = torch.empty(call.B, call.Hq, call.Sq, dtype=torch.float32, device=q.device)
    p = call.params(q, k, v, out, lse)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        bind_mod_buffers(call.module, call.score_mod, call.mask_mod, q.device)
        if call.use_decode():
            splits = int(call.options.get("num_splits", 0))
            if splits <= 0:
                sms = torch.cuda.get_device_properties(q.device).multi_processor_count
                splits = L.fa_decode_num_splits(p, sms)
            nbytes = L.fa_decode_workspace_bytes(p, splits)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
            _cabi.check(L.fa_decode(call.module.handle, p, splits, ws.data_ptr(), nbytes, stream))
        else:
            _cabi.check(L.fa_fwd(call.module.handle, p, stream))
    return out, lse


def _backward(call: _Call, q, k, v, out, lse, dout):
    L = _cabi.lib()
    check_status()
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = call.params(q, k, v, out, lse)
    nbytes = L.fa_bwd_workspace_bytes(p)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        bind_mod_buffers(call.module, call.score_mod, call.mask_mod, q.device)
        _cabi.check(L.fa_bwd(call.module.handle, p, _tensor(dout, call.layout), _tensor(dq, call.layout),
                             _tensor(dk, call.layout), _tensor(dv, call.layout), ws.data_ptr(), nbytes, stream))
    return dq, dk, dv


class _AttentionFn(torch.autograd.Function):
    """Forward saves (q, k, v, out, lse), the residuals of the reference's custom_vjp
    (flaxattention/kernel/attention.py:335); backward returns (dq, dk, dv)."""

    @staticmethod
    def forward(ctx, q, k, v, call: _Call):
        out, lse = _forward(call, q, k, v)
        ctx.call = call
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _backward(ctx.call, q, k, v, out, lse, dout)
        return dq, dk, dv, None


def _run(call: _Call, q, k, v):
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _AttentionFn.apply(q, k, v, call)
    return _forward(call, q, k, v)


def _as_cuda(x):
    """numpy -> CUDA tensor on the current device (host-to-device copy); tensors pass through."""
    if isinstance(x, np.ndarray):
        if not torch.cuda.is_available():
            raise RuntimeError("flaxattention_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        return torch.from_numpy(x).cuda(non_blocking=True), True
    return x, False


# --------------------------------------------------------------------------------------
# public API
# --------------------------------------------------------------------------------------
def flax_attention(
    query,
    key,
    value,
    score_mod: Optional[Callable] = None,
    block_mask: Optional[BlockMask] = None,
    scale: Optional[float] = None,
    enable_gqa: bool = False,
    return_lse: bool = False,
    kernel_options: Optional[Dict[str, Any]] = None,
    *,
    b_offset: int = 0,
    h_offset: int = 0,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Attention with a fused ``score_mod`` and a BlockMask, ``[B, H, S, D]`` layout.

    Returns the output in the input dtype and, with ``return_lse``, the natural-log
    logsumexp ``[B, Hq, Sq]`` in float32 (``-inf`` for fully masked rows, whose output is 0).
    ``kernel_options``: ``{"path": "fwd" | "decode", "num_splits": int, "round_scores": bool}``.
    For fp16 / bf16 inputs the scores are rounded to the input dtype before the scale, as in
    the reference's dense path (``jnp.matmul`` in the input dtype, core/attention.py:27);
    ``round_scores=False`` keeps the fp32 product like ``flax_attention_pallas`` does.
    ``b_offset`` / ``h_offset`` are the global indices of the first batch / head of a
    batch x heads shard; the mods see global indices.
    """
    query, from_np = _as_cuda(query)
    key, _ = _as_cuda(key)
    value, _ = _as_cuda(value)
    _validate_sdpa_input(query, key, value)
    _validate_embed_dim(query, key, value)
    if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
        raise NotImplementedError("NYI: query, key, and value must be 4D tensors")
    _validate_heads(query.shape[-3], key.shape[-3], enable_gqa)
    if score_mod is None:
        score_mod = _identity
    if scale is None:
        scale = 1.0 / math.sqrt(query.shape[-1])
    mask_mod = None if block_mask is None else block_mask.mask_mod
    call = _Call(query, key, value, score_mod, mask_mod, block_mask, scale, "bhsd", b_offset, h_offset,
                 kernel_options, round_scores=True)
    out, lse = _run(call, query, key, value)
    if from_np:
        out, lse = out.cpu().numpy(), lse.cpu().numpy()
    if return_lse:
        return out, lse
    return out


_BOUND_MODS: Dict[Tuple, Tuple] = {}


def _bind_other_buffers(fn: Callable, bufs: Tuple, is_score: bool) -> Callable:
    """``fn(..., *bufs)`` as a mod of the plain signature.  The reference passes the extra
    arrays as trailing arguments (core/attention.py:35-52); here they become tensors the mod
    closes over, which the tracer turns into device loads.  The wrapper is cached on the
    identity of the function and the buffers so that repeated calls reuse the compiled module."""
    if not bufs:
        return fn
    key = (id(fn), is_score) + tuple(id(b) for b in bufs)
    hit = _BOUND_MODS.get(key)
    if hit is not None and hit[0] is fn and len(hit[1]) == len(bufs) and all(a is b for a, b in zip(hit[1], bufs)):
        return hit[3]
    tens = tuple(b if isinstance(b, torch.Tensor) else torch.as_tensor(np.asarray(b)) for b in bufs)
    if is_score:
        def bound(score, b, h, q_idx, kv_idx):
            return fn(score, b, h, q_idx, kv_idx, *tens)
    else:
        def bound(b, h, q_idx, kv_idx):
            return fn(b, h, q_idx, kv_idx, *tens)
    if len(_BOUND_MODS) > 256:
        _BOUND_MODS.clear()
    _BOUND_MODS[key] = (fn, tuple(bufs), tens, bound)
    return bound


def math_attention(query, key, value, score_mod, block_mask: Tuple, scale, kernel_options=None,
                   score_mod_other_buffers: Tuple = (), mask_mod_other_buffers: Tuple = (), use_pallas: bool = False):
    """Signature of the reference's ``math_attention`` (core/attention.py:67-106): takes
    ``BlockMask.as_tuple()`` and returns ``(output, logsumexp / ln 2)``.  It runs the same
    fused kernels as ``flax_attention``; a dense score tensor is never built.
    ``score_mod_other_buffers`` / ``mask_mod_other_buffers`` are passed to the mods as trailing
    arguments, as the reference does (core/attention.py:35-52)."""
    mask_mod = block_mask[-1]
    score_mod = _bind_other_buffers(score_mod, tuple(score_mod_other_buffers), True)
    if mask_mod is not None:
        mask_mod = _bind_other_buffers(mask_mod, tuple(mask_mod_other_buffers), False)
    bm = BlockMask(*block_mask[:8], (block_mask[8], block_mask[9]), mask_mod)
    call = _Call(query, key, value, score_mod, mask_mod, bm, scale, "bhsd", 0, 0, kernel_options, round_scores=True)
    out, lse = _run(call, query, key, value)
    return out, lse / math.log(2.0)


def flax_attention_pallas(
    query,
    key,
    value,
    score_mod: Optional[Callable] = None,
    mask_mod: Optional[Callable] = None,
    block_q: int = 64,
    block_k: int = 64,
    sm_scale: Optional[float] = None,
    bhln: bool = True,
    enable_gqa: bool = False,
    *,
    block_mask: Optional[BlockMask] = None,
    return_lse: bool = False,
    b_offset: int = 0,
    h_offset: int = 0,
):
    """The reference's fused-kernel entry point.  ``bhln=True`` means ``[B, H, L, N]``
    inputs, ``False`` ``[B, L, H, N]``; either way the kernels read the tensors through
    strides, so the transposed copies the reference makes (core/attention.py:243-246, :312)
    do not happen.  ``block_q`` / ``block_k`` are accepted for compatibility; tile sizes are
    chosen by the library.  Beyond the reference: GQA is implemented (the reference only
    validates it), and an optional ``block_mask`` enables block skipping (its ``mask_mod``
    is used when ``mask_mod`` is not given)."""
    del block_q, block_k
    query, from_np = _as_cuda(query)
    key, _ = _as_cuda(key)
    value, _ = _as_cuda(value)
    _validate_sdpa_input(query, key, value)
    _validate_embed_dim(query, key, value)
    if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
        raise NotImplementedError("NYI: query, key, and value must be 4D tensors")
    h_axis = 1 if bhln else 2
    _validate_heads(query.shape[h_axis], key.shape[h_axis], enable_gqa)
    if sm_scale is None:
        sm_scale = 1 / math.sqrt(query.shape[-1])
    if score_mod is None:
        score_mod = _identity
    if mask_mod is None:
        mask_mod = block_mask.mask_mod if block_mask is not None else noop_mask
    call = _Call(query, key, value, score_mod, mask_mod, block_mask, sm_scale, "bhsd" if bhln else "bshd",
                 b_offset, h_offset, None)
    out, lse = _run(call, query, key, value)
    if from_np:
        out, lse = out.cpu().numpy(), lse.cpu().numpy()
    if return_lse:
        return out, lse
    return out
