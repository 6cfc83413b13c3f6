"""Scalar function namespace for writing score_mods / mask_mods (the role ``jax.numpy``
plays for the reference's mods, e.g. ``jnp.exp2`` in flaxattention/mods/alibi.py:16 and
``jnp.where`` in examples/benchmark.py:20-21).

Every function accepts the symbolic scalars a mod receives while it is lowered to device
code, and also numpy arrays and torch tensors, so that one mod definition serves both
the CUDA kernels and a dense CPU evaluation.
"""
from .modtrace import (  # noqa: F401
    abs, ceil, cos, exp, exp2, float32, floor, floor_divide, inf, int32, isinf, isnan,
    isneginf, log, log2, logical_and, logical_not, logical_or, maximum, minimum, ones,
    power, remainder, rsqrt, sigmoid, sign, sin, sqrt, tanh, where, zeros,
)
