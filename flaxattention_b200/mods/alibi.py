"""ALiBi score_mod (flaxattention/mods/alibi.py:5-20)."""
from .. import fnp


def generate_alibi_bias(H: int):
    """Returns the ALiBi score_mod for ``H`` heads: ``score + (q_idx - kv_idx) *
    2^(-8 (h+1) / H)``.  The sign follows the reference: the bias grows with the
    distance to past keys."""

    def alibi_mod(score, b, h, q_idx, kv_idx):
        scale = fnp.exp2(-((h + 1) * 8.0 / H))
        bias = (q_idx - kv_idx) * scale
        return score + bias

    return alibi_mod
