"""Attention-sink mask of StreamingLLM (flaxattention/masks/attention_sink.py:6-24)."""
from ..blockmask import and_masks, or_masks
from .causal import causal_mask


def generate_attention_sink(window_size: int, sink_size: int = 4):
    """Sliding window of ``window_size`` plus always-visible sink keys ``kv_idx <=
    sink_size`` (that is ``sink_size + 1`` keys, as the reference writes it), causal."""

    def sliding_window(b, h, q_idx, kv_idx):
        return q_idx - kv_idx <= window_size

    def attention_sink(b, h, q_idx, kv_idx):
        return kv_idx <= sink_size

    attention_sink_mask = and_masks(or_masks(attention_sink, sliding_window), causal_mask)
    attention_sink_mask.__name__ = f"attention_sink_{window_size}_{sink_size}"
    return attention_sink_mask
