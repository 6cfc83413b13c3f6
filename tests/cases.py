"""The mods of the stored golden cases, written for this package (mirrors of the torch
functions in tests/golden/make_golden.py)."""
from flaxattention_b200.blockmask import and_masks
from flaxattention_b200.masks import (causal_mask, generate_attention_sink, generate_causal_offset,
                                      generate_sliding_window)
from flaxattention_b200.mods import checkerboard, generate_alibi_bias


def head_dependent(b, h, q, kv):
    return kv <= q + 64 * h + 32 * b


def all_masked(b, h, q, kv):
    return (q < 0) & (kv < 0)


def fullmask(batch_idx, head_idx, q_idx, kv_idx):
    return False


# name -> (B, Hq, Hkv, Sq, Skv, D, score_mod, mask_mod)
ATTENTION_CASES = {
    "nomod": (4, 8, 8, 64, 64, 32, None, None),
    "decode_alibi": (4, 8, 8, 1, 64, 32, generate_alibi_bias(8), None),
    "gqa": (2, 8, 2, 64, 64, 32, None, None),
    "checkerboard": (2, 4, 4, 64, 96, 32, checkerboard, None),
    "cfg1": (2, 4, 4, 256, 256, 64, generate_alibi_bias(4), causal_mask),
    "sink_ragged": (1, 2, 2, 200, 333, 32, None, generate_attention_sink(40, 4)),
}

# name -> (mask_mod, B, H, Q_LEN, KV_LEN, BLOCK_SIZE)
TABLE_CASES = {
    "causal_256": (causal_mask, 2, 4, 256, 256, 128),
    "causal_2048": (causal_mask, 1, 1, 2048, 2048, 128),
    "sink_8192": (generate_attention_sink(1024, 4), 1, 1, 8192, 8192, 128),
    "window_2048_64": (generate_sliding_window(256), 1, 2, 2048, 2048, 64),
    "head_dependent": (head_dependent, 2, 3, 512, 512, 128),
    "all_masked": (all_masked, 1, 1, 64, 64, 128),
}
# Q_LEN < 128: Q_BLOCK_SIZE = Q_LEN (flaxattention/core/blockmask.py:440-441); ragged
# lengths: mask_mod is evaluated on the padded positions (:443-444).  Current torch differs
# on both, so there are no stored vectors; these are checked against the oracle only.
TABLE_CASES_SOURCE_ONLY = {
    "decode_sq1": (generate_causal_offset(16383), 1, 1, 1, 16384, 128),
    "decode_sq16": (generate_causal_offset(16384 - 16), 2, 2, 16, 16384, 128),
    "decode_sq64_literal_causal": (causal_mask, 1, 2, 64, 4096, 128),
    "short_q_tuple_block": (causal_mask, 1, 1, 100, 512, (64, 256)),
    "ragged": (causal_mask, 1, 2, 200, 300, 128),
    "rect_grid": (generate_sliding_window(300), 1, 2, 512, 1024, 128),
}
TABLE_KEYS = ("kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices",
              "q_num_blocks", "q_indices", "full_q_num_blocks", "full_q_indices")
