from .causal import causal_mask, generate_causal_offset
from .sliding_window import generate_sliding_window
from .attention_sink import generate_attention_sink

__all__ = ["causal_mask", "generate_causal_offset", "generate_sliding_window", "generate_attention_sink"]
