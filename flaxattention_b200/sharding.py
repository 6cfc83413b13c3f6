"""Batch x heads partitioning of an attention problem over the GPUs of one node.

Every (batch, head) pair is independent in the forward, the backward and the decode
kernels, so the path shards with no exchange step: each rank runs the same kernels on its
slice and no collective is needed.  The only cross-rank fact a rank needs is the GLOBAL
index of its first batch entry and head, because score_mod / mask_mod may read ``b`` and
``h`` (ALiBi's slope depends on ``h``, flaxattention/mods/alibi.py:16); these are passed to
the kernels as ``b_offset`` / ``h_offset``.  With GQA, heads are cut in whole kv groups.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class Shard:
    rank: int
    mesh: Tuple[int, int]          # (ranks along batch, ranks along heads)
    b: slice                       # batch entries of this rank
    hq: slice                      # query heads of this rank
    hkv: slice                     # kv heads of this rank

    @property
    def b_offset(self) -> int:
        return self.b.start

    @property
    def h_offset(self) -> int:
        return self.hq.start


def choose_mesh(world: int, B: int, Hkv: int) -> Tuple[int, int]:
    """Largest batch split that divides B, the rest over kv heads (e.g. 8 GPUs: B=8 -> 8x1,
    B=4 H=16 -> 4x2)."""
    if world <= 0:
        raise ValueError("world size must be positive")
    for nb in range(min(world, B), 0, -1):
        if world % nb == 0 and B % nb == 0:
            nh = world // nb
            if Hkv % nh == 0:
                return nb, nh
    raise ValueError(f"cannot partition B={B} x Hkv={Hkv} over {world} ranks in whole batch entries and kv heads")


def shard_for(rank: int, world: int, B: int, Hq: int, Hkv: int) -> Shard:
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    if Hq % Hkv:
        raise ValueError("Hq must be a multiple of Hkv")
    nb, nh = choose_mesh(world, B, Hkv)
    rb, rh = divmod(rank, nh)
    bs, hs = B // nb, Hkv // nh
    G = Hq // Hkv
    return Shard(rank, (nb, nh), slice(rb * bs, (rb + 1) * bs), slice(rh * hs * G, (rh + 1) * hs * G),
                 slice(rh * hs, (rh + 1) * hs))


def shard_attention(rank: int, world: int, query, key, value, score_mod=None, block_mask=None, **kw):
    """Runs this rank's slice of a global ``[B, H, S, D]`` problem and returns
    ``(shard, local_output)``.  ``block_mask`` holds the global tables; broadcast axes are
    kept whole."""
    from .attention import flax_attention

    sh = shard_for(rank, world, query.shape[0], query.shape[1], key.shape[1])
    bm = None if block_mask is None else block_mask.shard(sh.b, sh.hq)
    out = flax_attention(query[sh.b, sh.hq].contiguous(), key[sh.b, sh.hkv].contiguous(),
                         value[sh.b, sh.hkv].contiguous(), score_mod=score_mod, block_mask=bm,
                         enable_gqa=query.shape[1] != key.shape[1], b_offset=sh.b_offset, h_offset=sh.h_offset, **kw)
    return sh, out
