"""Attention steps whose inputs and results live in HOST memory.

``flax_attention`` / ``flax_attention_pallas`` work on device tensors.  A caller that holds
its activations in pinned host memory pays three serial phases per step when it uses them
directly: copy in, compute, copy out.  ``HostPipeline`` runs the same kernels through the
same C ABI but cuts the problem into chunks of (batch entry, head range) - every (batch,
head) pair is independent, the reason the path shards without a collective - and keeps the
copy engines and the SMs busy at the same time: chunk i+1 is on its way to the device while
chunk i is computed and the results of chunk i-1 travel back.  PCIe is full duplex, so the
step costs about the longer of the two copy directions plus the fill of the pipeline (the
first chunk's input copy and forward), instead of the sum of both directions and the kernels.

The whole step - every copy, every kernel launch and the dependencies between the four
streams - is recorded once into a CUDA graph per set of host buffers and replayed afterwards,
so a step costs one launch on the host however many chunks it has.  (Mods that read captured
tensors are launched eagerly instead: their address table is refreshed by a host-to-device
copy before each launch, which a graph would freeze.)

Each chunk is computed with its global batch and head offsets, so mods that read ``b`` or
``h`` see the same indices as in a single call and the results equal those of one call on the
whole problem (dQ of the tcgen05 backward to fp32 summation order, like any two runs of it).

All device buffers, BlockMask shards and parameter blocks are set up once in the
constructor; ``step`` allocates nothing.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Callable, List, Optional, Tuple

import torch

from . import _cabi
from .attention import _Call, _identity, check_status
from .blockmask import BlockMask, bind_mod_buffers, noop_mask
from .modtrace import lower_mods

_SLOTS = 3


class _Slot:
    pass


def _chunk_list(B: int, Hq: int, Hkv: int, chunks) -> List[Tuple[slice, slice, slice]]:
    """(batch slice, query-head slice, kv-head slice) per chunk.

    ``chunks="ramp"`` (the default): two small chunks of about an eighth of the batch, then
    chunks of about a quarter.  The pipeline is full once the first chunk's inputs are on the
    device and its forward has run, so a small first chunk shortens the fill, while larger
    later chunks keep the kernels efficient (a kernel over one batch entry has too few CTAs
    for 148 SMs and the kernels of successive chunks run one after the other).
    An integer asks for that many equal chunks: whole batch entries while there are enough of
    them, otherwise single batch entries cut into ranges of whole kv groups."""
    G = Hq // Hkv
    if chunks == "ramp":
        small, big = max(1, B // 8), max(1, B // 4)
        out, b0 = [], 0
        while b0 < B:
            n = min(small if len(out) < 2 else big, B - b0)
            out.append((slice(b0, b0 + n), slice(0, Hq), slice(0, Hkv)))
            b0 += n
        return out
    chunks = max(1, int(chunks))
    if chunks <= B:
        cb = (B + chunks - 1) // chunks
        return [(slice(b0, min(B, b0 + cb)), slice(0, Hq), slice(0, Hkv)) for b0 in range(0, B, cb)]
    parts = 1
    for cand in range(min(Hkv, chunks // B), 0, -1):
        if Hkv % cand == 0:
            parts = cand
            break
    hs = Hkv // parts
    return [(slice(b, b + 1), slice(j * hs * G, (j + 1) * hs * G), slice(j * hs, (j + 1) * hs))
            for b in range(B) for j in range(parts)]


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
                 scale: Optional[float] = None, chunks="ramp", b_offset: int = 0, h_offset: int = 0,
                 backward: bool = True, round_scores: bool = False, use_graph: bool = True):
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
        self.chunks = _chunk_list(B, Hq, Hkv, chunks)
        cb = max(c[0].stop - c[0].start for c in self.chunks)
        chq = max(c[1].stop - c[1].start for c in self.chunks)
        chk = max(c[2].stop - c[2].start for c in self.chunks)
        dev = self.dev
        L = _cabi.lib()
        self._L = L
        with torch.cuda.device(dev):
            # input copies, kernels, and two result streams (so that two copy engines share the
            # results of a chunk)
            self.s_in, self.s_cmp, self.s_out, self.s_out2 = (torch.cuda.Stream(dev) for _ in range(4))
            mk = lambda *s, dt=dtype: torch.empty(*s, dtype=dt, device=dev)  # noqa: E731
            self.slots = []
            for _ in range(min(_SLOTS, len(self.chunks))):
                s = _Slot()
                s.q, s.k, s.v = mk(cb, chq, Sq, D), mk(cb, chk, Skv, D), mk(cb, chk, Skv, Dv)
                s.o = mk(cb, chq, Sq, Dv)
                s.lse = mk(cb, chq, Sq, dt=torch.float32)
                if backward:
                    s.dout = torch.ones(cb, chq, Sq, Dv, dtype=dtype, device=dev)
                    s.dq, s.dk, s.dv = mk(cb, chq, Sq, D), mk(cb, chk, Skv, D), mk(cb, chk, Skv, Dv)
                self.slots.append(s)
            # one call description per (chunk, slot): shapes, mods, table shard, parameter block
            self.calls = []
            ws_bytes = 16
            for bs, hqs, hks in self.chunks:
                n, nq, nk = bs.stop - bs.start, hqs.stop - hqs.start, hks.stop - hks.start
                bm = None if block_mask is None else block_mask.shard(bs, hqs)
                per_slot = []
                for s in self.slots:
                    q, k, v, o, lse = s.q[:n, :nq], s.k[:n, :nk], s.v[:n, :nk], s.o[:n, :nq], s.lse[:n, :nq]
                    call = _Call(q, k, v, score_mod, mask_mod, bm, scale, "bhsd", b_offset + bs.start,
                                 h_offset + hqs.start, None, round_scores=round_scores)
                    p = call.params(q, k, v, o, lse)
                    ent = {"call": call, "p": p, "views": (q, k, v, o)}
                    if backward:
                        ws_bytes = max(ws_bytes, int(L.fa_bwd_workspace_bytes(C.byref(p))))
                        gv = (s.dout[:n, :nq], s.dq[:n, :nq], s.dk[:n, :nk], s.dv[:n, :nk])
                        ent["gviews"] = gv
                        ent["g"] = tuple(_cabi.FaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)) for t in gv)
                    per_slot.append(ent)
                self.calls.append(per_slot)
            self.ws_bytes = ws_bytes
            for s in self.slots:
                s.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            self.module = self.calls[0][0]["call"].module
            self._mods = (score_mod, mask_mod)
            nev = len(self.chunks)
            self.ev_in, self.ev_fwd, self.ev_cmp, self.ev_out, self.ev_out2 = (
                [torch.cuda.Event() for _ in range(nev)] for _ in range(5))
        has_buffers = bool(lower_mods(score_mod, None if mask_mod is noop_mask else mask_mod).buffers)
        self.use_graph = bool(use_graph) and not has_buffers
        self._graphs = {}
        self._warm = False

    def bytes_per_step(self):
        """(host-to-device, device-to-host) bytes one step moves."""
        B, Hq, Hkv, Sq, Skv, D, Dv = self.shape
        es = torch.empty(0, dtype=self.dtype).element_size()
        nq, nk, nv, no = B * Hq * Sq * D * es, B * Hkv * Skv * D * es, B * Hkv * Skv * Dv * es, B * Hq * Sq * Dv * es
        return nq + nk + nv, no + ((nq + nk + nv) if self.backward else 0)

    def step(self, hq, hk, hv, ho, hdq=None, hdk=None, hdv=None, hdout=None) -> None:
        backward = self.backward and hdq is not None
        check_status()
        args = (hq, hk, hv, ho, hdq, hdk, hdv, hdout)
        with torch.cuda.device(self.dev):
            if not self.use_graph:
                self._enqueue(torch.cuda.current_stream(self.dev), backward, *args)
                return
            if not self._warm:
                # the first pass runs eagerly: kernels are compiled, loaded and configured here,
                # none of which may happen while a stream is being captured
                self._enqueue(torch.cuda.current_stream(self.dev), backward, *args)
                self._warm = True
                return
            key = (backward,) + tuple(0 if t is None else t.data_ptr() for t in args)
            g = self._graphs.get(key)
            if g is None:
                if len(self._graphs) >= 8:
                    self._graphs.clear()
                g = torch.cuda.CUDAGraph()
                cap = torch.cuda.Stream(self.dev)
                cap.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.graph(g, stream=cap):
                    self._enqueue(torch.cuda.current_stream(self.dev), backward, *args)
                self._graphs[key] = g
            g.replay()

    def _enqueue(self, cur, backward, hq, hk, hv, ho, hdq, hdk, hdv, hdout) -> None:
        """Queues one step: side streams fork from `cur` and join it again at the end."""
        L, dev = self._L, self.dev
        ns = len(self.slots)
        bind_mod_buffers(self.module, self._mods[0], self._mods[1], dev)
        streams = (self.s_in, self.s_cmp, self.s_out, self.s_out2)
        for st in streams:
            st.wait_stream(cur)
        for i, (bs, hqs, hks) in enumerate(self.chunks):
            s = self.slots[i % ns]
            ent = self.calls[i][i % ns]
            q, k, v, o = ent["views"]
            with torch.cuda.stream(self.s_in):
                if i >= ns:
                    self.s_in.wait_event(self.ev_cmp[i - ns])  # the kernels of the chunk that held this slot are done
                q.copy_(hq[bs, hqs], non_blocking=True)
                k.copy_(hk[bs, hks], non_blocking=True)
                v.copy_(hv[bs, hks], non_blocking=True)
                if backward and hdout is not None:
                    ent["gviews"][0].copy_(hdout[bs, hqs], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            self.s_cmp.wait_event(self.ev_in[i])
            if i >= ns:
                self.s_cmp.wait_event(self.ev_out[i - ns])  # its results have left the slot
                self.s_cmp.wait_event(self.ev_out2[i - ns])
            raw = self.s_cmp.cuda_stream
            _cabi.check(L.fa_fwd(self.module.handle, C.byref(ent["p"]), raw))
            self.ev_fwd[i].record(self.s_cmp)
            if backward:
                g = ent["g"]
                _cabi.check(L.fa_bwd(self.module.handle, C.byref(ent["p"]), C.byref(g[0]), C.byref(g[1]),
                                     C.byref(g[2]), C.byref(g[3]), s.ws.data_ptr(), self.ws_bytes, raw))
            self.ev_cmp[i].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_fwd[i])  # the output leaves while the backward runs
                ho[bs, hqs].copy_(o, non_blocking=True)
                if backward:
                    self.s_out.wait_event(self.ev_cmp[i])
                    hdq[bs, hqs].copy_(ent["gviews"][1], non_blocking=True)
                self.ev_out[i].record(self.s_out)
            with torch.cuda.stream(self.s_out2):
                if backward:
                    self.s_out2.wait_event(self.ev_cmp[i])
                    hdk[bs, hks].copy_(ent["gviews"][2], non_blocking=True)
                    hdv[bs, hks].copy_(ent["gviews"][3], non_blocking=True)
                self.ev_out2[i].record(self.s_out2)
        for st in streams:
            cur.wait_stream(st)
