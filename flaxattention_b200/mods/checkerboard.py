"""Checkerboard score_mod of the reference's benchmark (examples/benchmark.py:17-22)."""
from .. import fnp


def checkerboard(score, batch, head, q_idx, k_idx):
    score = fnp.where((k_idx - q_idx) % 2 == 0, score * 0.5, score)
    score = fnp.where((k_idx - q_idx) % 2 == 1, score * 2.0, score)
    return score
