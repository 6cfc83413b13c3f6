"""Numpy restatement of the reference's BlockMask construction.  TEST INFRASTRUCTURE ONLY.

Follows flaxattention/core/blockmask.py:
  create_block_mask              :419-455  (B/H defaults, block sizes, Q_LEN<128 rule, rounding up)
  create_mask                    :277-322  (dense mask; a 5-argument function is a score_mod
                                            whose -inf results are the masked positions)
  _convert_mask_to_block_mask    :335-369  (block sums, partial / full grids)
  _dense_to_ordered              :57-64    (row sum; stable descending argsort)
  _ordered_to_dense / _transpose_ordered :30-54, :67-69  (q tables)

Pinning: the reference could not be run here (no JAX).  The kv tables are pinned against
torch.nn.attention.flex_attention.create_block_mask on CPU (the upstream code the reference
transcribes) through tests/golden/.  The bit-exact contract is the four kv tables.
"""
from __future__ import annotations

import inspect
from typing import Callable, Dict, Optional, Tuple, Union

import numpy as np


def _arity(fn) -> int:
    return sum(1 for p in inspect.signature(fn).parameters.values() if p.default is inspect.Parameter.empty)


def create_mask(mod_fn: Callable, B: Optional[int], H: Optional[int], Q_LEN: int, KV_LEN: int,
                b_offset: int = 0, h_offset: int = 0) -> np.ndarray:
    B = 1 if B is None else B
    H = 1 if H is None else H
    b = (np.arange(B, dtype=np.int32) + np.int32(b_offset)).reshape(B, 1, 1, 1)
    h = (np.arange(H, dtype=np.int32) + np.int32(h_offset)).reshape(1, H, 1, 1)
    m = np.arange(Q_LEN, dtype=np.int32).reshape(1, 1, Q_LEN, 1)
    n = np.arange(KV_LEN, dtype=np.int32).reshape(1, 1, 1, KV_LEN)
    if _arity(mod_fn) == 5:
        out = mod_fn(np.zeros((B, H, Q_LEN, KV_LEN), dtype=np.float32), b, h, m, n)
        mask = ~np.isneginf(np.asarray(out))
    else:
        mask = np.asarray(mod_fn(b, h, m, n)).astype(bool)
    return np.broadcast_to(mask, (B, H, Q_LEN, KV_LEN))


def dense_to_ordered(dense: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    dense = dense.astype(np.int32)
    num = dense.sum(axis=-1).astype(np.int32)
    idx = np.argsort(-dense, axis=-1, kind="stable").astype(np.int32)
    return num, idx


def ordered_to_dense(num: np.ndarray, idx: np.ndarray) -> np.ndarray:
    cols = idx.shape[-1]
    valid = np.arange(cols) < num[..., None]
    dense = np.zeros(idx.shape[:-1] + (cols + 1,), dtype=np.int32)
    tgt = np.where(valid, idx, cols)
    np.put_along_axis(dense, tgt, 1, axis=-1)
    return dense[..., :cols]


def block_grids(mask: np.ndarray, Q_BLOCK: int, KV_BLOCK: int) -> Tuple[np.ndarray, np.ndarray]:
    B, H, Q, KV = mask.shape
    assert Q % Q_BLOCK == 0 and KV % KV_BLOCK == 0
    m = mask.reshape(B, H, Q // Q_BLOCK, Q_BLOCK, KV // KV_BLOCK, KV_BLOCK).transpose(0, 1, 2, 4, 3, 5)
    s = m.sum(axis=(-2, -1), dtype=np.int64)
    full = s == Q_BLOCK * KV_BLOCK
    partial = (s > 0) & (s < Q_BLOCK * KV_BLOCK)
    return partial.astype(np.int8), full.astype(np.int8)


def create_block_mask_oracle(mask_mod: Callable, B: Optional[int], H: Optional[int], Q_LEN: int, KV_LEN: int,
                             BLOCK_SIZE: Union[int, Tuple[int, int]] = 128, b_offset: int = 0,
                             h_offset: int = 0) -> Dict[str, np.ndarray]:
    """Tables as a dict: kv_num_blocks, kv_indices, full_kv_num_blocks, full_kv_indices,
    q_num_blocks, q_indices, full_q_num_blocks, full_q_indices (true transposes),
    ref_q_num_blocks, ref_q_indices (the degenerate values the reference stores), BLOCK_SIZE."""
    B = 1 if B is None else B
    H = 1 if H is None else H
    if isinstance(BLOCK_SIZE, int):
        QB = KVB = BLOCK_SIZE
    else:
        QB, KVB = BLOCK_SIZE
    if Q_LEN < 128:
        QB = Q_LEN
    else:
        Q_LEN = (Q_LEN + QB - 1) // QB * QB
    KV_LEN = (KV_LEN + KVB - 1) // KVB * KVB
    # evaluate in head chunks so that big problems stay small in memory
    partial = np.zeros((B, H, Q_LEN // QB, KV_LEN // KVB), dtype=np.int8)
    full = np.zeros_like(partial)
    for b in range(B):
        for h in range(H):
            m = create_mask(mask_mod, 1, 1, Q_LEN, KV_LEN, b_offset + b, h_offset + h)
            p, f = block_grids(m, QB, KVB)
            partial[b, h], full[b, h] = p[0, 0], f[0, 0]
    kv_num, kv_idx = dense_to_ordered(partial)
    fkv_num, fkv_idx = dense_to_ordered(full)
    q_num, q_idx = dense_to_ordered(np.swapaxes(ordered_to_dense(kv_num, kv_idx), -1, -2))
    fq_num, fq_idx = dense_to_ordered(np.swapaxes(ordered_to_dense(fkv_num, fkv_idx), -1, -2))
    nq, nkv = partial.shape[-2:]
    ref_q_num = np.zeros((B, H, nkv), dtype=np.int32)
    ref_q_idx = np.broadcast_to(np.arange(nq, dtype=np.int32), (B, H, nkv, nq)).copy()
    return dict(kv_num_blocks=kv_num, kv_indices=kv_idx, full_kv_num_blocks=fkv_num, full_kv_indices=fkv_idx,
                q_num_blocks=q_num, q_indices=q_idx, full_q_num_blocks=fq_num, full_q_indices=fq_idx,
                ref_q_num_blocks=ref_q_num, ref_q_indices=ref_q_idx, BLOCK_SIZE=(QB, KVB),
                partial=partial, full=full)
