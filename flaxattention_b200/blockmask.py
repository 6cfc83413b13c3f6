"""BlockMask container and its construction on the GPU.

Mirrors flaxattention/core/blockmask.py: ``BlockMask`` (:72-237), ``create_block_mask``
(:419-455), ``and_masks`` / ``or_masks`` (:372-397), ``noop_mask`` (:20-27).  The dense
``[B,H,Q,KV]`` boolean mask the reference materialises (:277-322) is never built: a CUDA
kernel classifies every block directly from the lowered ``mask_mod`` and a second one
writes the ordered tables.

Table layout (all int32, on the CUDA device):
    kv_num_blocks [B,H,nQ], kv_indices [B,H,nQ,nKV]        blocks that need mask_mod
    full_kv_num_blocks, full_kv_indices                     blocks kept entirely
    q_num_blocks [B,H,nKV], q_indices [B,H,nKV,nQ], full_q_*   the same grid by kv block
Row order is the reference's (stable descending argsort of the 0/1 grid, :57-64): listed
blocks ascending, then the remaining block ids ascending.

Two deliberate differences from the reference, both on fields its own code never reads:
``BLOCK_SIZE`` holds the block sizes actually used (the reference always stores
(128, 128), :452-454), and the q-tables are the true transpose of the kv-tables (the
reference's ``_ordered_to_dense`` drops its scatter result, :46, so its q tables are
always ``num = 0, indices = arange``).  ``reference_q_tables`` reproduces those values.
"""
from __future__ import annotations

import collections
import functools
import operator
from typing import Callable, Optional, Tuple, Union

import torch

from . import _cabi
from .modtrace import lower_mods, mod_arity

_DEFAULT_SPARSE_BLOCK_SIZE = 128
_LARGE_SPARSE_BLOCK_SIZE = 1 << 30


def noop_mask(batch, head, token_q, token_kv):
    """Returns a noop mask_mod (everything visible)."""
    return True


def or_masks(*mask_mods: Callable) -> Callable:
    """Returns a mask_mod that's the union of provided mask_mods"""
    if not all(callable(arg) for arg in mask_mods):
        raise RuntimeError(f"All inputs should be callable mask_mods: {mask_mods}")

    def or_mask(b, h, q_idx, kv_idx):
        result = False
        for mask in mask_mods:
            result = result | mask(b, h, q_idx, kv_idx)
        return result

    return or_mask


def and_masks(*mask_mods: Callable) -> Callable:
    """Returns a mask_mod that's the intersection of provided mask_mods"""
    if not all(callable(arg) for arg in mask_mods):
        raise RuntimeError(f"All inputs should be callable mask_mods: {mask_mods}")

    def and_mask(b, h, q_idx, kv_idx):
        result = True
        for mask in mask_mods:
            result = result & mask(b, h, q_idx, kv_idx)
        return result

    return and_mask


def _dense_to_ordered(dense: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    dense = dense.to(torch.int32)
    num = dense.sum(dim=-1).to(torch.int32)
    idx = torch.argsort(dense, dim=-1, descending=True, stable=True).to(torch.int32)
    return num, idx


def _ordered_to_dense(num: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    rows, cols = idx.shape[-2], idx.shape[-1]
    dense = torch.zeros(*idx.shape[:-1], cols + 1, dtype=torch.int32, device=idx.device)
    valid = torch.arange(cols, device=idx.device) < num[..., None]
    tgt = torch.where(valid, idx.to(torch.int64), torch.full_like(idx, cols, dtype=torch.int64))
    dense.scatter_(-1, tgt, torch.ones_like(tgt, dtype=torch.int32))
    return dense[..., :cols]


def _transpose_ordered(num: torch.Tensor, idx: torch.Tensor):
    dense = _ordered_to_dense(num, idx)
    return _dense_to_ordered(dense.transpose(-1, -2).contiguous())


def reference_q_tables(kv_indices: torch.Tensor):
    """The q-table values the reference produces for any kv-tables of this shape:
    ``q_num_blocks = 0`` and ``q_indices = arange(nQ)`` (its scatter result is discarded,
    flaxattention/core/blockmask.py:46)."""
    *lead, n_q, n_kv = kv_indices.shape
    num = torch.zeros(*lead, n_kv, dtype=torch.int32, device=kv_indices.device)
    idx = torch.arange(n_q, dtype=torch.int32, device=kv_indices.device).expand(*lead, n_kv, n_q).contiguous()
    return num, idx


class BlockMask:
    kv_num_blocks: torch.Tensor
    kv_indices: torch.Tensor
    full_kv_num_blocks: Optional[torch.Tensor]
    full_kv_indices: Optional[torch.Tensor]
    q_num_blocks: Optional[torch.Tensor]
    q_indices: Optional[torch.Tensor]
    full_q_num_blocks: Optional[torch.Tensor]
    full_q_indices: Optional[torch.Tensor]
    BLOCK_SIZE: Tuple[int, int]
    mask_mod: Callable
    # mask_mod of every position as a bit matrix [1 or B, 1 or H, Q_LEN, words] (int32), or None;
    # not part of the reference's BlockMask: the kernels read it on partial tiles instead of
    # evaluating mask_mod there
    mask_bits: Optional[torch.Tensor] = None

    def __init__(self, kv_num_blocks, kv_indices, full_kv_num_blocks, full_kv_indices, q_num_blocks, q_indices,
                 full_q_num_blocks, full_q_indices, BLOCK_SIZE, mask_mod, mask_bits=None):
        if kv_indices.ndim < 2:
            raise RuntimeError("BlockMask must have at least 2 dimensions")
        assert kv_num_blocks is not None, "kv_num_blocks must be provided"
        assert kv_indices is not None, "kv_indices must be provided"
        assert q_num_blocks is not None, "q_num_blocks must be provided"
        assert q_indices is not None, "q_indices must be provided"
        assert (full_kv_num_blocks is None) == (
            full_kv_indices is None
        ), "full_kv_num_blocks and full_kv_indices must be both provided or omitted"
        assert (full_q_num_blocks is None) == (
            full_q_indices is None
        ), "full_q_num_blocks and full_q_indices must be both provided or omitted"
        self.kv_num_blocks = kv_num_blocks
        self.kv_indices = kv_indices
        self.full_kv_num_blocks = full_kv_num_blocks
        self.full_kv_indices = full_kv_indices
        self.q_num_blocks = q_num_blocks
        self.q_indices = q_indices
        self.full_q_num_blocks = full_q_num_blocks
        self.full_q_indices = full_q_indices
        self.BLOCK_SIZE = BLOCK_SIZE
        self.mask_mod = mask_mod
        self.mask_bits = mask_bits

    @classmethod
    def from_kv_blocks(cls, kv_num_blocks, kv_indices, full_kv_num_blocks=None, full_kv_indices=None,
                       BLOCK_SIZE: Union[int, Tuple[int, int]] = _DEFAULT_SPARSE_BLOCK_SIZE,
                       mask_mod: Optional[Callable] = None):
        if kv_indices.ndim < 2:
            raise RuntimeError("BlockMask must have at least 2 dimensions")
        assert (full_kv_num_blocks is None) == (
            full_kv_indices is None
        ), "full_kv_num_blocks and full_kv_indices must be both provided or omitted"
        q_num_blocks, q_indices = _transpose_ordered(kv_num_blocks, kv_indices)
        if full_kv_num_blocks is not None:
            full_q_num_blocks, full_q_indices = _transpose_ordered(full_kv_num_blocks, full_kv_indices)
        else:
            full_q_num_blocks, full_q_indices = None, None
        if isinstance(BLOCK_SIZE, int):
            BLOCK_SIZE = (BLOCK_SIZE, BLOCK_SIZE)
        mask_mod = mask_mod if mask_mod is not None else noop_mask
        return cls(kv_num_blocks, kv_indices, full_kv_num_blocks, full_kv_indices, q_num_blocks, q_indices,
                   full_q_num_blocks, full_q_indices, BLOCK_SIZE, mask_mod)

    def as_tuple(self, flatten: bool = True):
        """Returns a tuple of the attributes of the BlockMask (mask_mod last).

        Args:
            flatten (bool): If True, the (Q_BLOCK_SIZE, KV_BLOCK_SIZE) pair is flattened.
        """
        block_size = (self.BLOCK_SIZE[0], self.BLOCK_SIZE[1]) if flatten else (self.BLOCK_SIZE,)
        return (
            self.kv_num_blocks, self.kv_indices, self.full_kv_num_blocks, self.full_kv_indices,
            self.q_num_blocks, self.q_indices, self.full_q_num_blocks, self.full_q_indices,
            *block_size, self.mask_mod,
        )

    @property
    def shape(self):
        """Returns the shape of the mask."""
        *batch_dims, _, _ = self.kv_indices.shape
        q_length = self.kv_indices.shape[-2] * self.BLOCK_SIZE[0]
        kv_length = self.kv_indices.shape[-1] * self.BLOCK_SIZE[1]
        return tuple(list(batch_dims) + [q_length, kv_length])

    def numel(self):
        """Returns the number of elements (not accounting for sparsity) in the mask."""
        return functools.reduce(operator.mul, self.shape, 1)

    def sparsity(self) -> float:
        """Computes the percentage of blocks that are sparse (i.e. not computed)"""
        total_size = self.numel()
        computed_blocks = int(self.kv_num_blocks.sum().item())
        if self.full_kv_num_blocks is not None:
            computed_blocks += int(self.full_kv_num_blocks.sum().item())
        computed_size = computed_blocks * self.BLOCK_SIZE[0] * self.BLOCK_SIZE[1]
        return 100 * (1 - computed_size / total_size)

    def computed_blocks(self) -> int:
        """Number of (q block, kv block) pairs an attention call visits."""
        n = int(self.kv_num_blocks.sum().item())
        if self.full_kv_num_blocks is not None:
            n += int(self.full_kv_num_blocks.sum().item())
        return n

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)  # noqa: E731
        return BlockMask(mv(self.kv_num_blocks), mv(self.kv_indices), mv(self.full_kv_num_blocks),
                         mv(self.full_kv_indices), mv(self.q_num_blocks), mv(self.q_indices),
                         mv(self.full_q_num_blocks), mv(self.full_q_indices), self.BLOCK_SIZE, self.mask_mod,
                         mv(self.mask_bits))

    def shard(self, b_slice: slice, h_slice: slice) -> "BlockMask":
        """Tables of one batch x heads shard (broadcast axes are kept whole)."""
        def cut(t):
            if t is None:
                return None
            bs = b_slice if t.shape[0] != 1 else slice(None)
            hs = h_slice if t.shape[1] != 1 else slice(None)
            return t[bs, hs].contiguous()
        return BlockMask(cut(self.kv_num_blocks), cut(self.kv_indices), cut(self.full_kv_num_blocks),
                         cut(self.full_kv_indices), cut(self.q_num_blocks), cut(self.q_indices),
                         cut(self.full_q_num_blocks), cut(self.full_q_indices), self.BLOCK_SIZE, self.mask_mod,
                         cut(self.mask_bits))

    def __repr__(self):
        def shape_or_none(x):
            return tuple(x.shape) if x is not None else None

        return (
            f"BlockMask(\n"
            f"    kv_num_blocks={shape_or_none(self.kv_num_blocks)},\n"
            f"    kv_indices={shape_or_none(self.kv_indices)},\n"
            f"    full_kv_num_blocks={shape_or_none(self.full_kv_num_blocks)},\n"
            f"    full_kv_indices={shape_or_none(self.full_kv_indices)},\n"
            f"    q_num_blocks={shape_or_none(self.q_num_blocks)},\n"
            f"    q_indices={shape_or_none(self.q_indices)},\n"
            f"    full_q_num_blocks={shape_or_none(self.full_q_num_blocks)},\n"
            f"    full_q_indices={shape_or_none(self.full_q_indices)},\n"
            f"    BLOCK_SIZE={self.BLOCK_SIZE},\n"
            f"    shape={self.shape},\n"
            f"    sparsity={self.sparsity():.2f}%,\n"
            f"    mask_mod={self.mask_mod.__name__ if hasattr(self.mask_mod, '__name__') else self.mask_mod}\n"
            f")"
        )


def _create_empty_block_mask(query, key) -> BlockMask:
    """Default block mask: one block that spans the whole query and key range
    (flaxattention/core/blockmask.py:240-250)."""
    dev = query.device
    return BlockMask.from_kv_blocks(
        kv_num_blocks=torch.ones([1, 1, 1], dtype=torch.int32, device=dev),
        kv_indices=torch.zeros([1, 1, 1, 1], dtype=torch.int32, device=dev),
        BLOCK_SIZE=_LARGE_SPARSE_BLOCK_SIZE,
    )


def _round_up_to_multiple(x, multiple):
    return (x + multiple - 1) // multiple * multiple


_MODULES = {}


def module_for(score_mod: Optional[Callable], mask_mod: Optional[Callable]):
    """Lowered mods -> compiled-kernel module, cached per generated source."""
    if mask_mod is noop_mask:
        mask_mod = None
    ms = lower_mods(score_mod, mask_mod)
    m = _MODULES.get(ms.key)
    if m is None:
        m = _cabi.Module(ms.source)
        _MODULES[ms.key] = m
    return m


_DEVICE_BUFFERS = {}


def bind_mod_buffers(module, score_mod: Optional[Callable], mask_mod: Optional[Callable], device) -> None:
    """Hands the module the device addresses of the tensors the mods close over and index
    (the reference's score_mod_other_buffers / mask_mod_other_buffers,
    flaxattention/core/attention.py:22-23).  Tensors that live elsewhere (CPU, another GPU) are
    copied to `device` once per tensor version; the copies are kept while the mods are cached."""
    if mask_mod is noop_mask:
        mask_mod = None
    ms = lower_mods(score_mod, mask_mod)
    if not ms.buffers:
        return
    ptrs, keep = [], []
    for t in ms.buffers:
        if not isinstance(t, torch.Tensor):
            t = torch.as_tensor(t)
        if t.device != device:
            key = (id(t), t._version, str(device))
            hit = _DEVICE_BUFFERS.get(key)
            if hit is None or hit[0] is not t:
                if len(_DEVICE_BUFFERS) > 256:
                    _DEVICE_BUFFERS.clear()
                # same strides as the original: the load indices were built from them
                span = 1 + sum((d - 1) * st for d, st in zip(t.shape, t.stride()))
                flat = torch.as_strided(t, (span,), (1,)).to(device)
                hit = (t, flat)
                _DEVICE_BUFFERS[key] = hit
            t = hit[1]
        keep.append(t)
        ptrs.append(t.data_ptr())
    module.set_buffers(ptrs)
    module._bound_buffers = keep  # the addresses stay valid at least until the next binding


# finished tables of create_block_mask(..., _compile=True), least recently used first
_TABLE_CACHE: "collections.OrderedDict" = collections.OrderedDict()
_TABLE_CACHE_MAX = 64


def _require_cuda(device) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("flaxattention_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"flaxattention_b200 tensors must live on a CUDA device, got {dev}")
    return dev


_MASK_BITS_MAX_BYTES = 64 << 20


def _build_mask_bits(module, mask_mod, B, H, Q_LEN, KV_LEN, b_offset, h_offset, dev, force):
    """The bit matrix of ``mask_mod`` (see create_block_mask), or None.  Called with ``dev`` current
    and the module's captured buffers bound."""
    if force is False or mask_mod is noop_mask:
        return None
    ms = lower_mods(None, mask_mod)
    if ms.buffers and force is not True:
        return None
    # a mask whose device code never names b (h) is the same for every batch entry (head)
    import re
    m = re.search(r"fa_mask_mod\(int b, int h, int q, int kv\) \{(.*?)\n\}", ms.source, re.S)
    body = m.group(1) if m else "b h"
    reads_b, reads_h = re.search(r"\bb\b", body) is not None, re.search(r"\bh\b", body) is not None
    nb = B if reads_b else 1
    nh = H if reads_h else 1
    L = _cabi.lib()
    words = int(L.fa_mask_bits_row_words(KV_LEN))
    if force is not True and nb * nh * Q_LEN * words * 4 > _MASK_BITS_MAX_BYTES:
        return None
    if nb * nh > 65535 or Q_LEN > 65535:
        return None
    bits = torch.empty(nb, nh, Q_LEN, words, dtype=torch.int32, device=dev)
    _cabi.check(L.fa_mask_bits(module.handle, nb, nh, Q_LEN, KV_LEN, b_offset if reads_b else 0,
                               h_offset if reads_h else 0, bits.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return bits


def create_block_mask(
    mask_mod: Callable,
    B: Optional[int],
    H: Optional[int],
    Q_LEN: int,
    KV_LEN: int,
    BLOCK_SIZE: Union[int, Tuple[int, int]] = _DEFAULT_SPARSE_BLOCK_SIZE,
    _compile=False,
    device=None,
    b_offset: int = 0,
    h_offset: int = 0,
    _mask_bits: Optional[bool] = None,
) -> BlockMask:
    """Builds the BlockMask of ``mask_mod`` on the GPU.

    Same arguments as the reference.  The kernels are always compiled; ``_compile=True`` (the
    reference jits the construction so that repeated calls are cheap,
    flaxattention/core/blockmask.py:445-448) additionally keeps the finished tables, keyed by the
    lowered mask source, the shape, the block sizes, the offsets and the device, so a repeated
    call launches nothing.  Masks that read captured tensors are not kept (their contents may
    change between calls).  ``b_offset`` / ``h_offset`` give the global index of the first batch
    / head when the tables of one batch x heads shard are built.  A 5-argument function is
    treated as a score_mod whose ``-inf`` results mark masked positions.

    Next to the tables the mask itself is kept as a bit matrix (``BlockMask.mask_bits``, 1 bit per
    position where the reference's ``create_mask`` materialises a boolean,
    flaxattention/core/blockmask.py:277-322), one entry along batch / heads when ``mask_mod`` does
    not read ``b`` / ``h``: on the partial tiles the attention kernels read a row's words instead of
    evaluating ``mask_mod`` 128 times per row.  It is built when it takes at most 64 MiB and the mask
    reads no captured tensor (``_mask_bits=True`` / ``False`` forces it on or off).
    """
    if mod_arity(mask_mod) not in (4, 5):
        raise AssertionError("mask_mod must take (b, h, q_idx, kv_idx) or (score, b, h, q_idx, kv_idx)")
    if B is None:
        B = 1
    if H is None:
        H = 1
    if isinstance(BLOCK_SIZE, int):
        Q_BLOCK_SIZE = BLOCK_SIZE
        KV_BLOCK_SIZE = BLOCK_SIZE
    else:
        Q_BLOCK_SIZE, KV_BLOCK_SIZE = BLOCK_SIZE
    if Q_LEN < 128:
        Q_BLOCK_SIZE = Q_LEN
    else:
        Q_LEN = _round_up_to_multiple(Q_LEN, Q_BLOCK_SIZE)
    KV_LEN = _round_up_to_multiple(KV_LEN, KV_BLOCK_SIZE)
    dev = _require_cuda(device)
    nq, nkv = Q_LEN // Q_BLOCK_SIZE, KV_LEN // KV_BLOCK_SIZE
    module = module_for(None, mask_mod)
    cache_key = None
    if _compile:
        ms = lower_mods(None, None if mask_mod is noop_mask else mask_mod)
        if not ms.buffers:
            cache_key = (ms.key, B, H, Q_LEN, KV_LEN, Q_BLOCK_SIZE, KV_BLOCK_SIZE, int(b_offset), int(h_offset), str(dev))
            hit = _TABLE_CACHE.get(cache_key)
            if hit is not None:
                _TABLE_CACHE.move_to_end(cache_key)
                return BlockMask(*hit[:8], (Q_BLOCK_SIZE, KV_BLOCK_SIZE), mask_mod, hit[8])
    L = _cabi.lib()
    with torch.cuda.device(dev):
        mk = lambda *s: torch.empty(*s, dtype=torch.int32, device=dev)  # noqa: E731
        kv_num, kv_idx = mk(B, H, nq), mk(B, H, nq, nkv)
        fkv_num, fkv_idx = mk(B, H, nq), mk(B, H, nq, nkv)
        q_num, q_idx = mk(B, H, nkv), mk(B, H, nkv, nq)
        fq_num, fq_idx = mk(B, H, nkv), mk(B, H, nkv, nq)
        ws_bytes = L.fa_block_mask_workspace_bytes(B, H, Q_LEN, KV_LEN, Q_BLOCK_SIZE, KV_BLOCK_SIZE)
        ws = torch.empty(ws_bytes, dtype=torch.int8, device=dev)
        bind_mod_buffers(module, None, mask_mod, dev)
        _cabi.check(L.fa_block_mask(
            module.handle, B, H, Q_LEN, KV_LEN, Q_BLOCK_SIZE, KV_BLOCK_SIZE, b_offset, h_offset,
            kv_num.data_ptr(), kv_idx.data_ptr(), fkv_num.data_ptr(), fkv_idx.data_ptr(),
            q_num.data_ptr(), q_idx.data_ptr(), fq_num.data_ptr(), fq_idx.data_ptr(),
            ws.data_ptr(), ws_bytes, torch.cuda.current_stream(dev).cuda_stream))
        bits = _build_mask_bits(module, mask_mod, B, H, Q_LEN, KV_LEN, b_offset, h_offset, dev, _mask_bits)
    if cache_key is not None:
        _TABLE_CACHE[cache_key] = (kv_num, kv_idx, fkv_num, fkv_idx, q_num, q_idx, fq_num, fq_idx, bits)
        while len(_TABLE_CACHE) > _TABLE_CACHE_MAX:
            _TABLE_CACHE.popitem(last=False)
    return BlockMask(kv_num, kv_idx, fkv_num, fkv_idx, q_num, q_idx, fq_num, fq_idx,
                     (Q_BLOCK_SIZE, KV_BLOCK_SIZE), mask_mod, bits)
