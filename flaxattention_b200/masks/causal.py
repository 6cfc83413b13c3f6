"""Standard causal attention masking (flaxattention/masks/causal.py:4-5)."""


def causal_mask(b, h, q_idx, kv_idx):
    return q_idx >= kv_idx


def generate_causal_offset(offset: int):
    """Causal mask for a query block that sits at the END of the key range: query row
    ``q_idx`` is token ``q_idx + offset`` (decoding with ``offset = Skv - Sq``).  The
    reference's ``causal_mask`` compares raw indices, which for Sq=1 leaves a single
    visible key; this is the variant its decoding benchmark needs."""

    def causal_offset_mask(b, h, q_idx, kv_idx):
        return q_idx + offset >= kv_idx

    causal_offset_mask.__name__ = f"causal_offset_{offset}"
    return causal_offset_mask
