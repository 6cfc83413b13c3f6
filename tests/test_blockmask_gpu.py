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


# ---- the mask as a bit matrix (BlockMask.mask_bits) --------------------------------------------
def _unpack_bits(bits, kv_len):
    """[.., Q, words] int32 -> [.., Q, kv_len] bool."""
    w = bits.cpu().numpy().view(np.uint32)
    cols = np.arange(kv_len)
    return ((w[..., cols // 32] >> (cols % 32).astype(np.uint32)) & 1).astype(bool)


def test_mask_bits_equal_the_mask_of_the_oracle():
    from flaxattention_b200 import create_block_mask
    from flaxattention_b200.masks import causal_mask, generate_attention_sink
    from oracle.blockmask_oracle import create_mask as create_mask_oracle

    for mask, Q, KV in ((causal_mask, 256, 384), (generate_attention_sink(100, 4), 512, 512)):
        bm = create_block_mask(mask, 2, 3, Q, KV)
        assert bm.mask_bits is not None and tuple(bm.mask_bits.shape[:3]) == (1, 1, Q), "one entry: the mask reads neither b nor h"
        got = _unpack_bits(bm.mask_bits, KV)[0, 0]
        want = create_mask_oracle(mask, 1, 1, Q, KV)[0, 0]
        assert np.array_equal(got, want)
    # a mask that reads the head index keeps one entry per head; offsets are the global indices
    def per_head(b, h, q_idx, kv_idx):
        return (q_idx >= kv_idx) & ((kv_idx + h) % 3 != 0)
    bm = create_block_mask(per_head, 1, 4, 128, 200, h_offset=2)
    assert tuple(bm.mask_bits.shape[:2]) == (1, 4)
    # (KV_LEN is rounded up to whole blocks, as for the tables: 256 keys)
    want = create_mask_oracle(per_head, 1, 4, 128, 256, h_offset=2)[0]
    assert np.array_equal(_unpack_bits(bm.mask_bits, 256)[0], want)
    # a one-entry shard of a mask that reads b still sees its global batch index
    def per_batch(b, h, q_idx, kv_idx):
        return kv_idx <= q_idx + 32 * b
    bm = create_block_mask(per_batch, 1, 2, 128, 256, b_offset=3)
    want = create_mask_oracle(per_batch, 1, 1, 128, 256, b_offset=3)[0, 0]
    assert tuple(bm.mask_bits.shape[:2]) == (1, 1) and np.array_equal(_unpack_bits(bm.mask_bits, 256)[0, 0], want)


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_attention_is_the_same_with_and_without_mask_bits(D, dtype):
    """The kernels read the bit matrix on partial tiles instead of evaluating mask_mod: forward and
    gradients must not change by a bit (decode variant included)."""
    import flaxattention_b200 as fa
    from flaxattention_b200.masks import generate_attention_sink, generate_causal_offset

    torch.manual_seed(3)
    dev = torch.device("cuda", 0)
    mask = generate_attention_sink(200, 4)
    B, H, S = 2, 4, 640
    q, k, v = (torch.randn(B, H, S, D, device=dev, dtype=dtype, requires_grad=True) for _ in range(3))
    res = []
    for use in (True, False):
        bm = fa.create_block_mask(mask, B, H, S, S, _mask_bits=use)
        assert (bm.mask_bits is not None) == use
        out = fa.flax_attention(q, k, v, block_mask=bm)
        g = torch.autograd.grad(out.float().square().sum(), (q, k, v))
        res.append((out, *g))
    for a, b in zip(*res):
        assert torch.equal(a, b)
    if D == 64:
        sq = 48
        kk, vv = k.detach()[:, :, :, :].repeat(1, 1, 2, 1), v.detach().repeat(1, 1, 2, 1)  # Skv = 1280
        qq = q.detach()[:, :, :sq]
        m2 = generate_causal_offset(kk.shape[2] - sq)
        outs = [fa.flax_attention(qq, kk, vv, block_mask=fa.create_block_mask(m2, B, H, sq, kk.shape[2], _mask_bits=u))
                for u in (True, False)]
        assert torch.equal(outs[0], outs[1])
