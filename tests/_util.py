"""Shared helpers of the test-suite: seeded inputs and error measures."""
import numpy as np
import torch

DTYPES = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def normal(seed: int, shape, dtype=torch.float32) -> torch.Tensor:
    """N(0,1) tensor from a counter-based generator, so that every test case is
    reproducible independently of the order tests run in.  The reference's tests draw K, Q
    and V from PRNGKey(0), (1), (2) (tests/attention_test.py:32-40); the same seed
    assignment is used here."""
    g = np.random.Generator(np.random.Philox(seed))
    return torch.from_numpy(g.standard_normal(size=shape, dtype=np.float32)).to(dtype)


def qkv(B, Hq, Hkv, Sq, Skv, D, Dv=None, dtype=torch.float32):
    Dv = D if Dv is None else Dv
    k = normal(0, (B, Hkv, Skv, D), dtype)
    q = normal(1, (B, Hq, Sq, D), dtype)
    v = normal(2, (B, Hkv, Skv, Dv), dtype)
    return q, k, v


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.double() - b.double()).abs().max().item()


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max |a - ref| / max |ref|: the 'relative to an fp32 reference' measure for gradients."""
    d = (a.double() - ref.double()).abs().max().item()
    return d / max(ref.double().abs().max().item(), 1e-30)


def lse_err(lse: torch.Tensor, ref: torch.Tensor):
    """(max abs error over finite entries, whether the -inf patterns agree)."""
    fin = torch.isfinite(ref)
    same_inf = bool(torch.equal(torch.isneginf(lse), torch.isneginf(ref)))
    err = (lse[fin].double() - ref[fin].double()).abs().max().item() if fin.any() else 0.0
    return err, same_inf
