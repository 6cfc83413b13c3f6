"""flaxattention_b200: the flash-attention hot path of flaxattention, rebuilt for B200.

Export list follows flaxattention/__init__.py:11-22 (without the matplotlib visualiser).
"""
from .attention import check_status, flax_attention, flax_attention_pallas, math_attention
from .blockmask import BlockMask, and_masks, create_block_mask, noop_mask, or_masks
from .pipeline import HostPipeline
from . import fnp, masks, mods  # noqa: F401
from typing import Callable

_mask_mod_signature = Callable
_score_mod_signature = Callable

__all__ = [
    "math_attention",
    "flax_attention",
    "flax_attention_pallas",
    "BlockMask",
    "create_block_mask",
    "and_masks",
    "or_masks",
    "noop_mask",
    "_mask_mod_signature",
    "_score_mod_signature",
    "check_status",
    "HostPipeline",
    "fnp",
    "masks",
    "mods",
]
