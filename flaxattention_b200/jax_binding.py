"""JAX side of the ``jax.ffi`` binding: registers the handlers of ``csrc/ffi_shim.cc`` and wraps
them in the ``custom_vjp`` the reference builds around its Pallas launches
(flaxattention/kernel/attention.py:166-205, residuals ``(q, k, v, out, lse)`` :335, gradients
``(dq, dk, dv)`` :650).  A maintainer of the reference calls ``mha`` below where
``flax_attention_pallas`` calls the Pallas ``mha`` today (flaxattention/core/attention.py:298-309).

Needs JAX and the shim library (``python -m flaxattention_b200.csrc.build --ffi``).  The image this
package was developed on has neither, so nothing here has run; the torch / ctypes layer
(``attention.py``, ``_cabi.py``) is the tested binding of the same C ABI.
"""
from __future__ import annotations

import ctypes as C
import functools
import math
import os

from . import _cabi
from .modtrace import lower_mods

_HERE = os.path.dirname(os.path.abspath(__file__))
_SHIM = os.path.join(_HERE, "libflaxattn_ffi.so")
_registered = False


def _register():
    global _registered
    if _registered:
        return
    import jax

    _cabi.lib()  # the shim links against libflaxattn.so
    shim = C.CDLL(_SHIM, mode=C.RTLD_GLOBAL)
    for name in ("FaFwd", "FaBwd", "FaDecode", "FaBlockMask"):
        jax.ffi.register_ffi_target("fa_" + name[2:].lower(), jax.ffi.pycapsule(getattr(shim, name)), platform="CUDA")
    _registered = True


def _params_for(q, k, v, scale, bshd):
    """fa_attn_params with shapes only (no pointers): what the workspace queries need."""
    import jax.numpy as jnp

    p = _cabi.FaAttnParams()
    p.dtype = {jnp.dtype("float16"): _cabi.FA_F16, jnp.dtype("bfloat16"): _cabi.FA_BF16,
               jnp.dtype("float32"): _cabi.FA_F32}[jnp.dtype(q.dtype)]
    hs, ss = (2, 1) if bshd else (1, 2)
    p.B, p.Hq, p.Sq, p.D = q.shape[0], q.shape[hs], q.shape[ss], q.shape[3]
    p.Hkv, p.Skv, p.Dv = k.shape[hs], k.shape[ss], v.shape[3]
    p.scale = scale
    return p


@functools.lru_cache(maxsize=None)
def _module(score_mod, mask_mod):
    return _cabi.Module(lower_mods(score_mod, mask_mod).source)


def make_mha(score_mod=None, mask_mod=None, sm_scale=None, bshd=False, b_offset=0, h_offset=0):
    """Returns ``mha(q, k, v)`` for one (score_mod, mask_mod) pair: a ``jax.custom_vjp`` whose
    forward and backward are the ``fa_fwd`` / ``fa_bwd`` custom calls.  No BlockMask (every kv
    tile is visited and mask_mod applied), like the reference's fused entry point."""
    import jax
    import jax.numpy as jnp

    _register()
    module = _module(score_mod, mask_mod)
    empty = jnp.zeros((0,), jnp.int32)

    def attrs(scale):
        return dict(module=jnp.int64(module.handle.value), scale=jnp.float32(scale), bshd=jnp.int32(bshd),
                    has_tables=jnp.int32(0), q_block=jnp.int32(0), kv_block=jnp.int32(0), b_offset=jnp.int32(b_offset),
                    h_offset=jnp.int32(h_offset), flags=jnp.int32(0))

    def fwd(q, k, v):
        scale = 1.0 / math.sqrt(q.shape[-1]) if sm_scale is None else sm_scale
        rows = q.shape[:-1] if not bshd else (q.shape[0], q.shape[2], q.shape[1])
        out, lse = jax.ffi.ffi_call(
            "fa_fwd", (jax.ShapeDtypeStruct(q.shape[:-1] + v.shape[-1:], q.dtype), jax.ShapeDtypeStruct(rows, jnp.float32)))(
            q, k, v, empty, empty, empty, empty, **attrs(scale))
        return out, (q, k, v, out, lse)

    def bwd(res, dout):
        q, k, v, out, lse = res
        scale = 1.0 / math.sqrt(q.shape[-1]) if sm_scale is None else sm_scale
        ws = int(_cabi.lib().fa_bwd_workspace_bytes(C.byref(_params_for(q, k, v, scale, bshd))))
        dq, dk, dv, _ = jax.ffi.ffi_call(
            "fa_bwd", (jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct(k.shape, k.dtype),
                       jax.ShapeDtypeStruct(v.shape, v.dtype), jax.ShapeDtypeStruct((max(ws, 16),), jnp.uint8)))(
            q, k, v, out, lse, dout, *([empty] * 8), **attrs(scale))
        return dq, dk, dv

    @jax.custom_vjp
    def mha(q, k, v):
        return fwd(q, k, v)[0]

    mha.defvjp(fwd, bwd)
    return mha
