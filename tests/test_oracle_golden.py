"""Pins the CPU oracle (oracle/) against the stored golden vectors, which come from eager
torch flex_attention / create_block_mask / SDPA on CPU, the checker the reference's own
tests use (tests/attention_test.py, decimal=2).  CPU only."""
import os

import numpy as np
import pytest
import torch

from _util import max_abs, qkv
from cases import ATTENTION_CASES, TABLE_CASES, TABLE_KEYS, fullmask
from oracle.attention_oracle import attention_grads_oracle, flax_attention_oracle, flax_attention_oracle_chunked
from oracle.blockmask_oracle import create_block_mask_oracle

HERE = os.path.dirname(os.path.abspath(__file__))
ATT = np.load(os.path.join(HERE, "golden", "attention_golden.npz"))
TAB = np.load(os.path.join(HERE, "golden", "blockmask_golden.npz"))


@pytest.mark.parametrize("name", sorted(ATTENTION_CASES))
def test_attention_oracle_matches_golden(name):
    B, Hq, Hkv, Sq, Skv, D, score_mod, mask_mod = ATTENTION_CASES[name]
    stride = int(ATT[f"{name}.shape"][6])
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D)
    out, lse = flax_attention_oracle(q, k, v, score_mod, mask_mod)
    # fp32: the bar of the north star for fp32 results is 1e-5
    assert max_abs(out[:, :, ::stride], torch.from_numpy(ATT[f"{name}.out"])) <= 1e-5
    ref_lse = torch.from_numpy(ATT[f"{name}.lse"])
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    assert max_abs(lse[fin], ref_lse[fin]) <= 2e-5 * max(1.0, ref_lse[fin].abs().max().item())


def test_chunked_oracle_equals_dense():
    B, Hq, Hkv, Sq, Skv, D, score_mod, mask_mod = ATTENTION_CASES["cfg1"]
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D)
    o1, l1 = flax_attention_oracle(q, k, v, score_mod, mask_mod)
    o2, l2 = flax_attention_oracle_chunked(q, k, v, score_mod, mask_mod, chunk_bh=3)
    assert max_abs(o1, o2) <= 1e-6 and max_abs(l1, l2) <= 1e-5
    q, k, v = qkv(2, 8, 2, 32, 48, 16)
    o1, l1 = flax_attention_oracle(q, k, v, ATTENTION_CASES["decode_alibi"][6], None)
    o2, l2 = flax_attention_oracle_chunked(q, k, v, ATTENTION_CASES["decode_alibi"][6], None, chunk_bh=3)
    assert max_abs(o1, o2) <= 1e-6 and max_abs(l1, l2) <= 1e-5


def test_fully_masked_rows_give_zero_output_and_neginf_lse():
    # tests/attention_test.py:65-96 (test_fully_masked)
    q, k, v = qkv(4, 8, 8, 64, 64, 32)
    out, lse = flax_attention_oracle(q, k, v, None, fullmask)
    assert torch.count_nonzero(out) == 0 and bool(torch.isneginf(lse).all())


@pytest.mark.parametrize("name", ["grads_nomod", "grads_decode"])
def test_gradient_oracle_matches_sdpa_autograd(name):
    # tests/attention_test.py:385-430, :479-524 compare dQ with torch autograd
    B, Hq, Hkv, Sq, Skv, D, _ = (int(x) for x in ATT[f"{name}.shape"])
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D)
    out, lse, dq, dk, dv = attention_grads_oracle(q, k, v, torch.ones(B, Hq, Sq, D))
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert max_abs(got, torch.from_numpy(ATT[f"{name}.{key}"])) <= 1e-5


@pytest.mark.parametrize("name", sorted(TABLE_CASES))
def test_block_table_oracle_matches_golden(name):
    mask, B, H, Q, KV, bs = TABLE_CASES[name]
    t = create_block_mask_oracle(mask, B, H, Q, KV, bs)
    for key in TABLE_KEYS:
        assert np.array_equal(t[key], TAB[f"{name}.{key}"]), key
        assert t[key].dtype == np.int32


def test_block_statistics_of_the_benchmark_configurations():
    """Block counts the benchmark description quotes: causal 2048/128 -> 16 partial, 120
    full, 120 empty; sink(1024, 4) 8192/128 -> 175 partial, 420 full, 3501 empty."""
    t = create_block_mask_oracle(TABLE_CASES["causal_2048"][0], 1, 1, 2048, 2048)
    assert (t["kv_num_blocks"].sum(), t["full_kv_num_blocks"].sum()) == (16, 120)
    t = create_block_mask_oracle(TABLE_CASES["sink_8192"][0], 1, 1, 8192, 8192)
    assert (t["kv_num_blocks"].sum(), t["full_kv_num_blocks"].sum()) == (175, 420)


def test_short_query_rule():
    """Q_LEN < 128 makes the q block the whole query (core/blockmask.py:440-441): with the
    offset-causal decode mask every kv block but the last is full."""
    from cases import TABLE_CASES_SOURCE_ONLY

    t = create_block_mask_oracle(*TABLE_CASES_SOURCE_ONLY["decode_sq16"])
    assert t["BLOCK_SIZE"] == (16, 128) and t["kv_indices"].shape == (2, 2, 1, 128)
    assert (t["full_kv_num_blocks"] == 127).all() and (t["kv_num_blocks"] == 1).all()
    assert (t["kv_indices"][..., 0] == 127).all()
    t = create_block_mask_oracle(*TABLE_CASES_SOURCE_ONLY["decode_sq1"])
    assert (t["full_kv_num_blocks"] == 128).all() and (t["kv_num_blocks"] == 0).all()


def test_ragged_lengths_are_classified_on_padded_positions():
    from cases import TABLE_CASES_SOURCE_ONLY

    t = create_block_mask_oracle(*TABLE_CASES_SOURCE_ONLY["ragged"])
    # q block 1 (rows 128..255 after padding) x kv block 0 is entirely below the diagonal
    assert t["full_kv_num_blocks"][0, 0].tolist() == [0, 1]
    assert t["kv_num_blocks"][0, 0].tolist() == [1, 1]
    assert t["kv_indices"].shape == (1, 2, 2, 3)


def test_reference_q_tables_are_degenerate():
    t = create_block_mask_oracle(TABLE_CASES["causal_256"][0], 2, 4, 256, 256)
    assert not t["ref_q_num_blocks"].any()
    assert np.array_equal(t["ref_q_indices"][0, 0], np.array([[0, 1], [0, 1]], dtype=np.int32))
