"""Sliding-window causal mask (flaxattention/masks/sliding_window.py:7-22)."""
from ..blockmask import and_masks
from .causal import causal_mask


def generate_sliding_window(window_size: int):
    """Keys at most ``window_size`` positions behind the query are visible (so
    ``window_size + 1`` keys), future keys are masked."""

    def sliding_window(b, h, q_idx, kv_idx):
        return q_idx - kv_idx <= window_size

    sliding_window_mask = and_masks(sliding_window, causal_mask)
    sliding_window_mask.__name__ = f"sliding_window_{window_size}"
    return sliding_window_mask
