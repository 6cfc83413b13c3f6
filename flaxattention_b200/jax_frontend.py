"""jaxpr front end of the mod lowering, for mods written with ``jax.numpy``.

The reference's mods are JAX functions (flaxattention/mods/alibi.py:15-18, masks/*.py, the
``@jax.jit`` checkerboard of examples/benchmark.py:16-26) that it vmaps and jits
(flaxattention/core/common.py:41-81).  ``modtrace`` records a mod by calling it with symbolic
scalars, which covers mods written with plain operators, numpy, torch or ``fnp``; a mod that
calls ``jnp`` functions rejects those symbols.  Such a mod is traced by JAX itself instead:
``jax.make_jaxpr`` on scalar arguments gives a flat list of primitive applications, and this
module replays that list on ``modtrace.Sym`` values, inlining nested jaxprs (``pjit``,
``custom_jvp_call``, ``closed_call``).  The result is the same expression graph, so CUDA
lowering, the symbolic derivative and the affine detection are shared with the tracer.

Needs JAX; machines without it never import this module (``modtrace.lower_mods`` falls back to
it only when the symbolic call fails and ``jax`` is importable).
"""
from __future__ import annotations

from typing import Callable, Dict, List

import numpy as np

from . import modtrace as mt


def _unary(name):
    return lambda x, **kw: getattr(mt, name)(x)


def _convert(x, new_dtype=None, **kw):
    kind = np.dtype(new_dtype).kind
    if kind == "f":
        return mt.float32(x)
    if kind in "iu":
        return mt.int32(x)
    if kind == "b":
        return x != 0 if not (isinstance(x, mt.Sym) and x.dtype == mt.B1) else x
    raise NotImplementedError(f"convert_element_type to {new_dtype}")


def _integer_pow(x, y=None, **kw):
    out = x
    for _ in range(abs(int(y)) - 1):
        out = out * x
    return out if y > 0 else 1.0 / out


def _select_n(which, *cases, **kw):
    # select_n(pred, on_false, on_true) for a boolean predicate
    if len(cases) != 2:
        raise NotImplementedError("select_n with more than two cases")
    return mt.where(which, cases[1], cases[0])


_PRIMS: Dict[str, Callable] = {
    "add": lambda a, b, **kw: a + b, "sub": lambda a, b, **kw: a - b, "mul": lambda a, b, **kw: a * b,
    "div": lambda a, b, **kw: a / b if _is_float(a, b) else _trunc_div(a, b), "rem": lambda a, b, **kw: _c_rem(a, b),
    "neg": lambda a, **kw: -a, "abs": lambda a, **kw: mt.abs(a), "sign": _unary("sign"),
    "max": lambda a, b, **kw: mt.maximum(a, b), "min": lambda a, b, **kw: mt.minimum(a, b),
    "lt": lambda a, b, **kw: a < b, "le": lambda a, b, **kw: a <= b, "gt": lambda a, b, **kw: a > b,
    "ge": lambda a, b, **kw: a >= b, "eq": lambda a, b, **kw: a == b, "ne": lambda a, b, **kw: a != b,
    "and": lambda a, b, **kw: a & b, "or": lambda a, b, **kw: a | b, "xor": lambda a, b, **kw: a ^ b, "not": lambda a, **kw: ~a,
    "exp": _unary("exp"), "exp2": _unary("exp2"), "log": _unary("log"), "tanh": _unary("tanh"), "logistic": _unary("sigmoid"),
    "sqrt": _unary("sqrt"), "rsqrt": _unary("rsqrt"), "sin": _unary("sin"), "cos": _unary("cos"), "erf": lambda a, **kw: mt.Sym(mt.unary("erf", mt._lift(a))),
    "floor": _unary("floor"), "ceil": _unary("ceil"), "pow": lambda a, b, **kw: a ** b, "integer_pow": _integer_pow,
    "select_n": _select_n, "convert_element_type": _convert, "stop_gradient": lambda a, **kw: a, "copy": lambda a, **kw: a,
    "squeeze": lambda a, **kw: a, "reshape": lambda a, *_, **kw: a, "broadcast_in_dim": lambda a, *_, **kw: a,
}


def _is_float(*xs) -> bool:
    return any((isinstance(x, mt.Sym) and x.dtype == mt.F32) or isinstance(x, float) for x in xs)


def _trunc_div(a, b):
    # lax.div on integers truncates towards zero; the floor division of the operators rounds down
    q = a // b
    return mt.where(((a % b) != 0) & ((a < 0) != (b < 0)), q + 1, q)


def _c_rem(a, b):
    # lax.rem takes the sign of the dividend (C semantics); jnp.remainder is built from it
    if _is_float(a, b):
        return a - b * mt.where((a / b) >= 0, mt.floor(a / b), mt.ceil(a / b))
    return a - _trunc_div(a, b) * b


def _run_jaxpr(jaxpr, consts: List, args: List):
    env = {}

    def read(v):  # a Literal carries its value, a Var is looked up
        return v.val if hasattr(v, "val") else env[v]

    for var, c in zip(jaxpr.constvars, consts):
        arr = np.asarray(c)
        if arr.ndim != 0:
            raise NotImplementedError("mods over captured jax arrays: close over a torch tensor or numpy array "
                                      "and index it with the traced indices instead")
        env[var] = arr.item()
    for var, a in zip(jaxpr.invars, args):
        env[var] = a
    for eqn in jaxpr.eqns:
        ins = [read(v) for v in eqn.invars]
        name = eqn.primitive.name
        inner = eqn.params.get("jaxpr") or eqn.params.get("call_jaxpr")
        if inner is not None and name in ("pjit", "closed_call", "core_call", "custom_jvp_call", "custom_vjp_call", "remat"):
            closed = inner if hasattr(inner, "jaxpr") else None
            outs = _run_jaxpr(closed.jaxpr if closed else inner, list(closed.consts) if closed else [], ins)
        else:
            fn = _PRIMS.get(name)
            if fn is None:
                raise NotImplementedError(f"jax primitive '{name}' has no lowering to a device expression")
            outs = fn(*ins, **eqn.params)
            if not isinstance(outs, (list, tuple)):
                outs = [outs]
        for var, o in zip(eqn.outvars, outs):
            env[var] = o
    return [read(v) for v in jaxpr.outvars]


def trace_with_jax(fn: Callable, kind: str) -> "mt.TracedMod":
    """TracedMod of a score_mod (kind 'score') or mask_mod ('mask') written with jax.numpy."""
    import jax
    import jax.numpy as jnp

    i32 = jnp.int32(0)
    if kind == "score" or mt.mod_arity(fn) == 5:
        closed = jax.make_jaxpr(fn)(jnp.float32(0), i32, i32, i32, i32)
    else:
        closed = jax.make_jaxpr(fn)(i32, i32, i32, i32)

    def run():
        s, b, h, q, kv = mt._leaf_syms()
        if kind == "score":
            (out,) = _run_jaxpr(closed.jaxpr, list(closed.consts), [s, b, h, q, kv])
            return mt.cast(mt._lift(out), mt.F32)
        if mt.mod_arity(fn) == 5:  # a score_mod used as a mask: -inf marks masked positions
            (out,) = _run_jaxpr(closed.jaxpr, list(closed.consts), [mt.Sym(mt._B.const(0.0, mt.F32)), b, h, q, kv])
            return mt.unary("not", mt.unary("isneginf", mt.cast(mt._lift(out), mt.F32)))
        (out,) = _run_jaxpr(closed.jaxpr, list(closed.consts), [b, h, q, kv])
        return mt.cast(mt._lift(out), mt.B1)

    return mt._traced(None, run, kind)
