from .alibi import generate_alibi_bias
from .checkerboard import checkerboard

__all__ = ["generate_alibi_bias", "checkerboard"]
