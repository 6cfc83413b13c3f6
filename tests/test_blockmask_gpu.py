"""GPU parity of create_block_mask: the four kv tables must be bit-exact with the oracle
and with the stored vectors; the q tables must be the true transposes."""
import os

import numpy as np
import pytest
import torch

from cases import TABLE_CASES, TABLE_CASES_SOURCE_ONLY, TABLE_KEYS
from oracle.blockmask_oracle import create_block_mask_oracle

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
TAB = np.load(os.path.join(HERE, "golden", "blockmask_golden.npz"))


def _gpu_tables(mask, B, H, Q, KV, bs, **kw):
    from flaxattention_b200 import create_block_mask

    bm = create_block_mask(mask, B, H, Q, KV, BLOCK_SIZE=bs, **kw)
    torch.cuda.synchronize()
    return bm, {k: getattr(bm, k).cpu().numpy() for k in TABLE_KEYS}


@pytest.mark.parametrize("name", sorted(TABLE_CASES))
def test_tables_match_golden_and_oracle(name):
    mask, B, H, Q, KV, bs = TABLE_CASES[name]
    bm, got = _gpu_tables(mask, B, H, Q, KV, bs)
    want = create_block_mask_oracle(mask, B, H, Q, KV, bs)
    for k in TABLE_KEYS:
        assert got[k].dtype == np.int32
        assert np.array_equal(got[k], TAB[f"{name}.{k}"]), f"{k} differs from the stored vector"
        assert np.array_equal(got[k], want[k]), f"{k} differs from the oracle"
    assert bm.BLOCK_SIZE == want["BLOCK_SIZE"]


@pytest.mark.parametrize("name", sorted(TABLE_CASES_SOURCE_ONLY))
def test_tables_match_oracle(name):
    mask, B, H, Q, KV, bs = TABLE_CASES_SOURCE_ONLY[name]
    bm, got = _gpu_tables(mask, B, H, Q, KV, bs)
    want = create_block_mask_oracle(mask, B, H, Q, KV, bs)
    for k in TABLE_KEYS:
        assert np.array_equal(got[k], want[k]), k
    assert bm.BLOCK_SIZE == want["BLOCK_SIZE"]


def test_none_batch_and_heads_broadcast():
    from flaxattention_b200.masks import causal_mask

    bm, got = _gpu_tables(causal_mask, None, None, 512, 512, 128)
    assert got["kv_indices"].shape == (1, 1, 4, 4)
    want = create_block_mask_oracle(causal_mask, None, None, 512, 512)
    assert np.array_equal(got["kv_num_blocks"], want["kv_num_blocks"])
    assert abs(bm.sparsity() - 100 * (1 - 10 / 16)) < 1e-9
    assert "BlockMask(" in repr(bm) and bm.shape == (1, 1, 512, 512)


def test_shard_offsets_equal_slices_of_the_global_tables():
    """Tables built for one batch x heads shard (b_offset / h_offset) are the corresponding
    slices of the global tables."""
    from cases import head_dependent

    _, full = _gpu_tables(head_dependent, 4, 6, 512, 512, 128)
    _, part = _gpu_tables(head_dependent, 2, 3, 512, 512, 128, b_offset=2, h_offset=3)
    for k in TABLE_KEYS:
        assert np.array_equal(part[k], full[k][2:4, 3:6]), k


def test_score_mod_can_define_the_mask():
    """A 5-argument function is a score_mod whose -inf marks masked positions
    (flaxattention/core/blockmask.py:303-315)."""
    from flaxattention_b200 import fnp
    from flaxattention_b200.masks import causal_mask

    def neginf_future(score, b, h, q, kv):
        return fnp.where(q >= kv, score, -fnp.inf)

    _, got = _gpu_tables(neginf_future, 1, 2, 384, 384, 128)
    want = create_block_mask_oracle(causal_mask, 1, 2, 384, 384)
    for k in TABLE_KEYS:
        assert np.array_equal(got[k], want[k]), k


def test_from_kv_blocks_transposes_on_device():
    from flaxattention_b200 import BlockMask
    from flaxattention_b200.blockmask import reference_q_tables
    from flaxattention_b200.masks import generate_sliding_window

    mask = generate_sliding_window(200)
    _, got = _gpu_tables(mask, 1, 2, 1024, 1024, 128)
    dev = torch.device("cuda")
    bm = BlockMask.from_kv_blocks(*(torch.from_numpy(got[k]).to(dev) for k in TABLE_KEYS[:4]), BLOCK_SIZE=128,
                                  mask_mod=mask)
    for k in TABLE_KEYS[4:]:
        assert np.array_equal(getattr(bm, k).cpu().numpy(), got[k]), k
    num, idx = reference_q_tables(bm.kv_indices)
    assert not num.any() and idx.shape == bm.q_indices.shape
    assert len(bm.as_tuple()) == 11 and bm.as_tuple()[-1] is mask


def test_determinism():
    from flaxattention_b200.masks import generate_attention_sink

    _, a = _gpu_tables(generate_attention_sink(1024, 4), 2, 2, 4096, 4096, 128)
    _, b = _gpu_tables(generate_attention_sink(1024, 4), 2, 2, 4096, 4096, 128)
    for k in TABLE_KEYS:
        assert np.array_equal(a[k], b[k])
