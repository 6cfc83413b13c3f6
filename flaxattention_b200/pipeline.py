"""Attention steps whose inputs and results live in HOST memory.

``flax_attention`` / ``flax_attention_pallas`` work on device tensors.  A caller that holds
its activations in pinned host memory pays three serial phases per step when it uses them
directly: copy in, compute, copy out.  ``HostPipeline`` runs the same kernels through the
same C ABI but cuts the problem into chunks of batch entries (every (batch, head) pair is
independent, the reason the path shards without a collective) and keeps three streams busy:
chunk i+1 is on its way to the device while chunk i is computed and the results of chunk
i-1 travel back.  PCIe is full duplex, so the step costs about the longer of the two copy
directions instead of their sum plus the kernels.

Each chunk is computed with its global batch offset, so mods that read ``b`` see the same
indices as in a single call and the results equal those of one call on the whole batch
(dQ of the tcgen05 backward to fp32 summation order, like any two runs of it).

All device buffers, BlockMask shards and parameter blocks are set up once in the
constructor; ``step`` allocates nothing.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Callable, List, Optional

import torch

from . import _cabi
from .attention import _Call, _identity, check_status
from .blockmask import BlockMask, bind_mod_buffers, noop_mask

_SLOTS = 3


class _Slot:
    pass


class HostPipeline:
    """Forward (+ backward) of one attention problem ``[B, H, S, D]`` from pinned host buffers.

    ``step(hq, hk, hv, ho, hdq=None, hdk=None, hdv=None, hdout=None)``: the ``h*`` arguments are
    pinned host tensors of the full problem; with gradient buffers given the backward runs too
    (``hdout=None`` differentiates ``out.sum()``, i.e. dO = 1).  Work is queued behind the
    current stream and the current stream waits for it, so events recorded around ``step``
    time it and a following ``synchronize`` makes the host buffers valid.
    """

    def __init__(self, B: int, Hq: int, Hkv: int, Sq: int, Skv: int, D: int, Dv: Optional[int] = None, *,
                 dtype=torch.float16, device=None, score_mod: Optional[Callable] = None,
                 mask_mod: Optional[Callable] = None, block_mask: Optional[BlockMask] = None,
                 scale: Optional[float] = None, chunks: int = 4, b_offset: int = 0, h_offset: int = 0,
                 backward: bool = True, round_scores: bool = False):
        if not torch.cuda.is_available():
            raise RuntimeError("flaxattention_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        Dv = D if Dv is None else Dv
        self.shape = (B, Hq, Hkv, Sq, Skv, D, Dv)
        self.dtype = dtype
        self.backward = backward
        if score_mod is None:
            score_mod = _identity
        if mask_mod is None:
            mask_mod = block_mask.mask_mod if block_mask is not None else noop_mask
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        chunks = max(1, min(int(chunks), B))
        cb = (B + chunks - 1) // chunks
        self.chunks: List[slice] = [slice(b0, min(B, b0 + cb)) for b0 in range(0, B, cb)]
        dev = self.dev
        L = _cabi.lib()
        self._L = L
        with torch.cuda.device(dev):
            self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
            mk = lambda *s, dt=dtype: torch.empty(*s, dtype=dt, device=dev)  # noqa: E731
            self.slots = []
            for _ in range(min(_SLOTS, len(self.chunks))):
                s = _Slot()
                s.q, s.k, s.v = mk(cb, Hq, Sq, D), mk(cb, Hkv, Skv, D), mk(cb, Hkv, Skv, Dv)
                s.o = mk(cb, Hq, Sq, Dv)
                s.lse = mk(cb, Hq, Sq, dt=torch.float32)
                if backward:
                    s.dout = torch.ones(cb, Hq, Sq, Dv, dtype=dtype, device=dev)
                    s.dq, s.dk, s.dv = mk(cb, Hq, Sq, D), mk(cb, Hkv, Skv, D), mk(cb, Hkv, Skv, Dv)
                self.slots.append(s)
            # one call description per (chunk, slot): shapes, mods, table shard, parameter block
            self.calls = []
            ws_bytes = 16
            for ch in self.chunks:
                n = ch.stop - ch.start
                bm = None if block_mask is None else block_mask.shard(ch, slice(0, Hq))
                per_slot = []
                for s in self.slots:
                    q, k, v, o, lse = s.q[:n], s.k[:n], s.v[:n], s.o[:n], s.lse[:n]
                    call = _Call(q, k, v, score_mod, mask_mod, bm, scale, "bhsd", b_offset + ch.start, h_offset,
                                 None, round_scores=round_scores)
                    p = call.params(q, k, v, o, lse)
                    ent = {"call": call, "p": p, "n": n}
                    if backward:
                        ws_bytes = max(ws_bytes, int(L.fa_bwd_workspace_bytes(C.byref(p))))
                        ent["g"] = tuple(_cabi.FaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
                                         for t in (s.dout[:n], s.dq[:n], s.dk[:n], s.dv[:n]))
                    per_slot.append(ent)
                self.calls.append(per_slot)
            self.ws_bytes = ws_bytes
            for s in self.slots:
                s.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            self.module = self.calls[0][0]["call"].module
            self._mods = (score_mod, mask_mod)
            nev = len(self.chunks)
            self.ev_in = [torch.cuda.Event() for _ in range(nev)]
            self.ev_cmp = [torch.cuda.Event() for _ in range(nev)]
            self.ev_out = [torch.cuda.Event() for _ in range(nev)]

    def bytes_per_step(self):
        """(host-to-device, device-to-host) bytes one step moves."""
        B, Hq, Hkv, Sq, Skv, D, Dv = self.shape
        es = torch.empty(0, dtype=self.dtype).element_size()
        nq, nk, nv, no = B * Hq * Sq * D * es, B * Hkv * Skv * D * es, B * Hkv * Skv * Dv * es, B * Hq * Sq * Dv * es
        return nq + nk + nv, no + ((nq + nk + nv) if self.backward else 0)

    def step(self, hq, hk, hv, ho, hdq=None, hdk=None, hdv=None, hdout=None) -> None:
        backward = self.backward and hdq is not None
        check_status()
        L, dev = self._L, self.dev
        cur = torch.cuda.current_stream(dev)
        ns = len(self.slots)
        with torch.cuda.device(dev):
            bind_mod_buffers(self.module, self._mods[0], self._mods[1], dev)
            for st in (self.s_in, self.s_cmp, self.s_out):
                st.wait_stream(cur)
            for i, ch in enumerate(self.chunks):
                s = self.slots[i % ns]
                ent = self.calls[i][i % ns]
                n = ent["n"]
                with torch.cuda.stream(self.s_in):
                    if i >= ns:
                        self.s_in.wait_event(self.ev_cmp[i - ns])  # the kernels of the chunk that held this slot are done
                    s.q[:n].copy_(hq[ch], non_blocking=True)
                    s.k[:n].copy_(hk[ch], non_blocking=True)
                    s.v[:n].copy_(hv[ch], non_blocking=True)
                    if backward and hdout is not None:
                        s.dout[:n].copy_(hdout[ch], non_blocking=True)
                    self.ev_in[i].record(self.s_in)
                self.s_cmp.wait_event(self.ev_in[i])
                if i >= ns:
                    self.s_cmp.wait_event(self.ev_out[i - ns])  # its results have left the slot
                raw = self.s_cmp.cuda_stream
                _cabi.check(L.fa_fwd(self.module.handle, C.byref(ent["p"]), raw))
                if backward:
                    g = ent["g"]
                    _cabi.check(L.fa_bwd(self.module.handle, C.byref(ent["p"]), C.byref(g[0]), C.byref(g[1]),
                                         C.byref(g[2]), C.byref(g[3]), s.ws.data_ptr(), self.ws_bytes, raw))
                self.ev_cmp[i].record(self.s_cmp)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.ev_cmp[i])
                    ho[ch].copy_(s.o[:n], non_blocking=True)
                    if backward:
                        hdq[ch].copy_(s.dq[:n], non_blocking=True)
                        hdk[ch].copy_(s.dk[:n], non_blocking=True)
                        hdv[ch].copy_(s.dv[:n], non_blocking=True)
                    self.ev_out[i].record(self.s_out)
            for st in (self.s_in, self.s_cmp, self.s_out):
                cur.wait_stream(st)
