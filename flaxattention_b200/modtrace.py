"""Lowering of user ``score_mod`` / ``mask_mod`` callables to CUDA device-function fragments.

The reference evaluates the mods by ``jax.vmap`` over (kv, q, h, b)
(flaxattention/core/common.py:41-81) on the dense score tensor, and inside its Pallas
kernel on (block_q, block_k) index spans (flaxattention/kernel/attention.py:83-93).
Here a mod is called ONCE with symbolic scalars; every operator applied to them is
recorded into a small SSA expression graph (int32 / float32 / bool scalars).  That
graph has three back ends:

* ``to_cuda``      - text of a ``__device__ __forceinline__`` function that the runtime
                     compiler splices into the attention kernel templates;
* ``evaluate``     - a numpy evaluator (used by the tests to check the tracer);
* ``derivative``   - the symbolic derivative with respect to the score argument, which
                     plays the role of ``jax.grad(score_mod)``
                     (flaxattention/core/attention.py:286).

Integer ``%`` and ``//`` follow Python / ``jnp.remainder`` / ``jnp.floor_divide``
semantics (result takes the sign of the divisor, division rounds toward -inf).
Python scalars are weakly typed the way JAX treats them: ``int32 * 8.0`` is float32,
``int32 + 1`` stays int32, ``/`` always gives float32.
"""
from __future__ import annotations

import hashlib
import inspect
import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

I32, F32, B1 = "i32", "f32", "b1"

_LEAVES = ("score", "b", "h", "q", "kv")
_UNARY_F = (
    "exp", "exp2", "log", "log2", "sqrt", "rsqrt", "tanh", "sigmoid", "sin", "cos",
    "floor", "ceil", "erf",
)


class Expr:
    """One node of the expression graph (hash-consed, immutable)."""

    __slots__ = ("op", "dtype", "args", "value", "_key")

    def __init__(self, op: str, dtype: str, args: Tuple["Expr", ...] = (), value=None):
        self.op = op
        self.dtype = dtype
        self.args = args
        self.value = value
        self._key = (op, dtype, tuple(id(a) for a in args), value if op in ("const", "load") else None)

    def __repr__(self):
        if self.op == "const":
            return f"{self.value!r}:{self.dtype}"
        if not self.args:
            return self.op
        return f"{self.op}({', '.join(map(repr, self.args))})"


class _Builder:
    """Hash-consing constructor with light algebraic simplification."""

    def __init__(self):
        self._table: Dict[tuple, Expr] = {}

    def _mk(self, op, dtype, args=(), value=None) -> Expr:
        if op == "const":
            if dtype == F32:
                v = float(np.float32(value))
                key = ("const", dtype, np.float32(v).tobytes())
            elif dtype == I32:
                v = int(np.int64(value).astype(np.int32)) if not isinstance(value, int) else _wrap_i32(value)
                key = ("const", dtype, v)
            else:
                v = bool(value)
                key = ("const", dtype, v)
            e = self._table.get(key)
            if e is None:
                e = Expr("const", dtype, (), v)
                self._table[key] = e
            return e
        key = (op, dtype, tuple(id(a) for a in args), value if op == "load" else None)
        e = self._table.get(key)
        if e is None:
            e = Expr(op, dtype, tuple(args), value if op == "load" else None)
            self._table[key] = e
        return e

    def const(self, value, dtype) -> Expr:
        return self._mk("const", dtype, value=value)

    def leaf(self, name) -> Expr:
        return self._mk(name, F32 if name == "score" else I32)


def _wrap_i32(v: int) -> int:
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v & 0x80000000 else v


_B = _Builder()


def _depends_on_leaves(e: Expr, leaves, memo=None) -> bool:
    if memo is None:
        memo = {}
    r = memo.get(id(e))
    if r is None:
        r = e.op in leaves or any(_depends_on_leaves(a, leaves, memo) for a in e.args)
        memo[id(e)] = r
    return r


def _is_const(e: Expr, v=None) -> bool:
    if e.op != "const":
        return False
    return True if v is None else e.value == v


# --------------------------------------------------------------------------------------
# typed constructors
# --------------------------------------------------------------------------------------
def _is_bit(e: Expr) -> bool:
    """True when the int32 expression can only be 0 or 1."""
    if e.dtype != I32:
        return False
    if e.op == "const":
        return e.value in (0, 1)
    if e.op == "and":
        return _is_const(e.args[0], 1) or _is_const(e.args[1], 1) or (_is_bit(e.args[0]) and _is_bit(e.args[1]))
    if e.op in ("or", "xor"):
        return _is_bit(e.args[0]) and _is_bit(e.args[1])
    if e.op == "cast_i32":
        return e.args[0].dtype == B1
    return False


def _parity(e: Expr) -> Expr:
    """e & 1 with the mask pushed through +, -, negation: the low bit of a sum is the xor of
    the low bits.  This separates the q and kv contributions of expressions like
    (kv - q) % 2, so that a kernel can evaluate the kv part per column at compile time."""
    if e.op == "const":
        return _B.const(e.value & 1, I32)
    if e.op in ("add", "sub") and e.dtype == I32:
        a, b = _parity(e.args[0]), _parity(e.args[1])
        if _is_const(a, 0):
            return b
        if _is_const(b, 0):
            return a
        if a.op == "const" and b.op == "const":
            return _B.const(a.value ^ b.value, I32)
        return _B._mk("xor", I32, (a, b))
    if e.op == "neg" and e.dtype == I32:
        return _parity(e.args[0])
    if _is_bit(e):
        return e
    return _B._mk("and", I32, (e, _B.const(1, I32)))


_UNARY_OPS = ("neg", "not", "abs", "isneginf", "isinf", "isnan", "sign") + _UNARY_F
_BINARY_OPS = ("add", "sub", "mul", "div", "floordiv", "rem", "pow", "min", "max", "and", "or", "xor", "shl", "shr",
               "lt", "le", "gt", "ge", "eq", "ne")


def _rebuild(e: Expr, args) -> Expr:
    if e.op in _UNARY_OPS:
        return unary(e.op, args[0])
    if e.op in _BINARY_OPS:
        return binary(e.op, args[0], args[1])
    if e.op == "select":
        return select(args[0], args[1], args[2])
    if e.op.startswith("cast_"):
        return cast(args[0], e.dtype)
    if e.op == "load":
        return _B._mk("load", e.dtype, (args[0],), e.value)
    raise NotImplementedError(e.op)


def _assume(e: Expr, cond: Expr, value: bool, memo=None) -> Expr:
    """e with the boolean node `cond` replaced by a constant, re-simplified."""
    if memo is None:
        memo = {}
    if e is cond:
        return _B.const(value, B1)
    if not e.args:
        return e
    got = memo.get(id(e))
    if got is not None:
        return got
    new_args = tuple(_assume(a, cond, value, memo) for a in e.args)
    r = e if all(x is y for x, y in zip(new_args, e.args)) else _rebuild(e, new_args)
    memo[id(e)] = r
    return r


def cast(e: Expr, dtype: str) -> Expr:
    if e.dtype == dtype:
        return e
    if e.op == "const":
        if dtype == B1:
            return _B.const(e.value != 0, B1)
        if dtype == I32:
            return _B.const(int(e.value), I32)
        return _B.const(float(e.value), F32)
    return _B._mk("cast_" + dtype, dtype, (e,))


def _promote(a: Expr, b: Expr) -> Tuple[Expr, Expr, str]:
    """Result type of an arithmetic op on two typed operands."""
    if F32 in (a.dtype, b.dtype):
        t = F32
    elif I32 in (a.dtype, b.dtype):
        t = I32
    else:
        t = B1
    return cast(a, t), cast(b, t), t


def binary(op: str, a: Expr, b: Expr) -> Expr:
    if op in ("and", "or", "xor"):
        a, b, t = _promote(a, b)
        if t == F32:
            raise TypeError(f"bitwise '{op}' is not defined for float operands")
        if t == I32 and op == "and":
            if _is_const(b, 1) and a.op in ("add", "sub", "neg", "const"):
                return _parity(a)
            if _is_const(a, 1) and b.op in ("add", "sub", "neg", "const"):
                return _parity(b)
        if t == B1:
            if op == "and":
                if _is_const(a):
                    return b if a.value else a
                if _is_const(b):
                    return a if b.value else b
            if op == "or":
                if _is_const(a):
                    return a if a.value else b
                if _is_const(b):
                    return b if b.value else a
        return _B._mk(op, t, (a, b))
    if op in ("lt", "le", "gt", "ge", "eq", "ne"):
        a, b, t = _promote(a, b)
        if t == B1:
            a, b = cast(a, I32), cast(b, I32)
        if op in ("eq", "ne") and t == I32:
            if a.op == "const" and b.op != "const":
                a, b = b, a
            if b.op == "const" and _is_bit(a) and a.op != "const":
                # a is 0 or 1: every test against a constant is `a == 0`, its negation, or constant
                is_zero = _B._mk("eq", B1, (a, _B.const(0, I32)))
                if b.value not in (0, 1):
                    return _B.const(op == "ne", B1)
                if (op == "eq") == (b.value == 0):
                    return is_zero
                return unary("not", is_zero)
        return _B._mk(op, B1, (a, b))
    if op in ("shl", "shr"):
        a, b = cast(a, I32), cast(b, I32)
        return _B._mk(op, I32, (a, b))
    a, b, t = _promote(a, b)
    if t == B1:
        a, b, t = cast(a, I32), cast(b, I32), I32
    if op == "div":
        a, b, t = cast(a, F32), cast(b, F32), F32
    if op == "pow":
        a, b, t = cast(a, F32), cast(b, F32), F32
    # light simplification; keeps derivative graphs small
    if op == "add":
        if _is_const(a, 0):
            return b
        if _is_const(b, 0):
            return a
    elif op == "sub":
        if _is_const(b, 0):
            return a
    elif op == "mul":
        if t == F32:
            # (x * y) * c -> x * (y * c) when y does not vary along a score row (no score, no kv):
            # the kernels can then hoist y * c out of their per-element loops
            for u, c in ((a, b), (b, a)):
                if c.op == "const" and u.op == "mul" and u.dtype == F32:
                    for x, y in ((u.args[0], u.args[1]), (u.args[1], u.args[0])):
                        if y.op != "const" and not _depends_on_leaves(y, ("score", "kv")) and _depends_on_leaves(x, ("score", "kv")):
                            return binary("mul", x, binary("mul", y, c))
        if _is_const(a, 1):
            return b
        if _is_const(b, 1):
            return a
        if _is_const(a, 0) or _is_const(b, 0):
            return _B.const(0, t)
    elif op == "div":
        if _is_const(b, 1):
            return a
    if t == I32 and op in ("rem", "floordiv") and b.op == "const" and b.value > 0 and (b.value & (b.value - 1)) == 0:
        # Python semantics for a positive power-of-two divisor are exactly the two's-complement
        # mask / arithmetic shift: x % 2^k == x & (2^k - 1), x // 2^k == x >> k
        if b.value == 1:
            return _B.const(0, I32) if op == "rem" else a
        if op == "rem":
            return binary("and", a, _B.const(b.value - 1, I32))
        return _B._mk("shr", I32, (a, _B.const(b.value.bit_length() - 1, I32)))
    if a.op == "const" and b.op == "const":
        folded = _fold_binary(op, a.value, b.value, t)
        if folded is not None:
            return _B.const(folded, t)
    return _B._mk(op, t, (a, b))


def _fold_binary(op, x, y, t):
    try:
        if t == F32:
            x32, y32 = np.float32(x), np.float32(y)
            with np.errstate(all="ignore"):
                if op == "add":
                    return float(x32 + y32)
                if op == "sub":
                    return float(x32 - y32)
                if op == "mul":
                    return float(x32 * y32)
                if op == "div":
                    return float(x32 / y32)
                if op == "min":
                    return float(np.minimum(x32, y32))
                if op == "max":
                    return float(np.maximum(x32, y32))
            return None
        if op == "add":
            return _wrap_i32(x + y)
        if op == "sub":
            return _wrap_i32(x - y)
        if op == "mul":
            return _wrap_i32(x * y)
        if op == "floordiv" and y != 0:
            return _wrap_i32(x // y)
        if op == "rem" and y != 0:
            return _wrap_i32(x % y)
        if op == "min":
            return min(x, y)
        if op == "max":
            return max(x, y)
    except Exception:
        return None
    return None


def unary(op: str, a: Expr) -> Expr:
    if op == "neg":
        if a.dtype == B1:
            a = cast(a, I32)
        if a.op == "const":
            return _B.const(-a.value, a.dtype)
        return _B._mk("neg", a.dtype, (a,))
    if op == "not":
        if a.dtype == F32:
            raise TypeError("'~' is not defined for float operands")
        if a.op == "const" and a.dtype == B1:
            return _B.const(not a.value, B1)
        if a.op == "not" and a.dtype == B1:
            return a.args[0]
        return _B._mk("not", a.dtype, (a,))
    if op == "abs":
        if a.dtype == B1:
            return cast(a, I32)
        return _B._mk("abs", a.dtype, (a,))
    if op in ("isneginf", "isinf", "isnan"):
        return _B._mk(op, B1, (cast(a, F32),))
    if op == "sign":
        return _B._mk(op, a.dtype if a.dtype != B1 else I32, (a if a.dtype != B1 else cast(a, I32),))
    if op in _UNARY_F:
        a = cast(a, F32)
        if a.op == "const" and op in ("exp2", "exp", "log", "log2", "sqrt"):
            with np.errstate(all="ignore"):
                f = {"exp2": np.exp2, "exp": np.exp, "log": np.log, "log2": np.log2, "sqrt": np.sqrt}[op]
                return _B.const(float(f(np.float32(a.value))), F32)
        return _B._mk(op, F32, (a,))
    raise ValueError(f"unknown unary op {op}")


def select(c: Expr, a: Expr, b: Expr) -> Expr:
    c = cast(c, B1)
    a, b, t = _promote(a, b)
    if c.op == "const":
        return a if c.value else b
    if c.op == "not":
        c, a, b = c.args[0], b, a
    # inside the arms the condition is known
    a = _assume(a, c, True)
    b = _assume(b, c, False)
    a, b, t = _promote(a, b)
    if a is b:
        return a
    return _B._mk("select", t, (c, a, b))


# --------------------------------------------------------------------------------------
# the tracer value
# --------------------------------------------------------------------------------------
def _lift(x) -> Expr:
    if isinstance(x, Sym):
        return x.e
    if isinstance(x, Expr):
        return x
    if isinstance(x, (bool, np.bool_)):
        return _B.const(bool(x), B1)
    if isinstance(x, (int, np.integer)):
        return _B.const(int(x), I32)
    if isinstance(x, (float, np.floating)):
        return _B.const(float(x), F32)
    if isinstance(x, np.ndarray) and x.ndim == 0:
        return _lift(x.item())
    try:  # 0-d torch tensors captured as constants
        import torch

        if isinstance(x, torch.Tensor) and x.ndim == 0:
            return _lift(x.item())
    except ImportError:  # pragma: no cover
        pass
    raise TypeError(
        f"cannot use a value of type {type(x).__name__} inside a score_mod/mask_mod trace; "
        "only Python scalars and the traced arguments are supported"
    )


# --------------------------------------------------------------------------------------
# captured buffers: tensors a mod closes over and indexes with traced values
# (score_mod_other_buffers / mask_mod_other_buffers of flaxattention/core/attention.py:22-23,
#  :35-52; in the reference they are jaxpr constants, here the tensors the closure holds)
# --------------------------------------------------------------------------------------
MAX_MOD_BUFFERS = 8
_ELEM_TYPES = {
    "torch.int32": ("i32", I32), "torch.int64": ("i64", I32), "torch.uint8": ("u8", I32), "torch.bool": ("u8", B1),
    "torch.float32": ("f32", F32),
    "int32": ("i32", I32), "int64": ("i64", I32), "uint8": ("u8", I32), "bool": ("u8", B1), "float32": ("f32", F32),
}
_TRACE_BUFFERS: Optional[List[object]] = None  # buffers of the mod pair being traced


def _buffer_load(buf, index) -> "Sym":
    """``buf[index]`` with traced indices: registers the tensor and records a load node.  The
    linear index is built from the tensor's strides; out-of-range indices (rows and keys of the
    padding of a ragged tile reach the mods too) are clamped by the generated code."""
    if _TRACE_BUFFERS is None:
        raise TypeError("a tensor can only be indexed with a traced value while a mod is being lowered")
    et = _ELEM_TYPES.get(str(buf.dtype))
    if et is None:
        raise TypeError(f"captured buffers of dtype {buf.dtype} are not supported (int32, int64, uint8, bool, float32 are)")
    idx = index if isinstance(index, tuple) else (index,)
    shape = tuple(int(d) for d in buf.shape)
    if len(idx) != len(shape):
        raise TypeError(f"a captured buffer of {len(shape)} dimensions needs {len(shape)} indices, got {len(idx)}")
    if hasattr(buf, "stride") and callable(buf.stride):
        strides = tuple(int(x) for x in buf.stride())
    else:
        strides = tuple(int(x // buf.itemsize) for x in buf.strides)
    numel = 1
    for d in shape:
        numel *= d
    if numel == 0 or numel >= (1 << 31):
        raise TypeError("captured buffers must hold between 1 and 2^31-1 elements")
    span = 1 + sum((d - 1) * st for d, st in zip(shape, strides))
    k = None
    for i, b in enumerate(_TRACE_BUFFERS):
        if b is buf:
            k = i
    if k is None:
        if len(_TRACE_BUFFERS) >= MAX_MOD_BUFFERS:
            raise TypeError(f"at most {MAX_MOD_BUFFERS} captured buffers per (score_mod, mask_mod) pair")
        _TRACE_BUFFERS.append(buf)
        k = len(_TRACE_BUFFERS) - 1
    lin = _B.const(0, I32)
    for i, st in zip(idx, strides):
        e = cast(_lift(i), I32)
        lin = binary("add", lin, binary("mul", e, _B.const(st, I32)))
    return Sym(_B._mk("load", et[1], (lin,), (k, span, et[0])))


def _bin(op):
    def f(self, other):
        try:
            return Sym(binary(op, self.e, _lift(other)))
        except TypeError:
            return NotImplemented

    def r(self, other):
        try:
            return Sym(binary(op, _lift(other), self.e))
        except TypeError:
            return NotImplemented

    return f, r


class Sym:
    """Symbolic scalar handed to a mod while it is traced."""

    __slots__ = ("e",)
    __array_priority__ = 1000

    def __init__(self, e: Expr):
        self.e = e

    @property
    def dtype(self):
        return {I32: np.dtype("int32"), F32: np.dtype("float32"), B1: np.dtype("bool")}[self.e.dtype]

    shape = ()
    ndim = 0

    __add__, __radd__ = _bin("add")
    __sub__, __rsub__ = _bin("sub")
    __mul__, __rmul__ = _bin("mul")
    __truediv__, __rtruediv__ = _bin("div")
    __floordiv__, __rfloordiv__ = _bin("floordiv")
    __mod__, __rmod__ = _bin("rem")
    __pow__, __rpow__ = _bin("pow")
    __and__, __rand__ = _bin("and")
    __or__, __ror__ = _bin("or")
    __xor__, __rxor__ = _bin("xor")
    __lshift__, __rlshift__ = _bin("shl")
    __rshift__, __rrshift__ = _bin("shr")
    __lt__, _ = _bin("lt")
    __le__, _ = _bin("le")
    __gt__, _ = _bin("gt")
    __ge__, _ = _bin("ge")
    __eq__, _ = _bin("eq")  # type: ignore[assignment]
    __ne__, _ = _bin("ne")  # type: ignore[assignment]
    __hash__ = None  # type: ignore[assignment]

    def __neg__(self):
        return Sym(unary("neg", self.e))

    def __pos__(self):
        return self

    def __invert__(self):
        return Sym(unary("not", self.e))

    def __abs__(self):
        return Sym(unary("abs", self.e))

    def __bool__(self):
        raise TypeError(
            "the truth value of a traced value is not known while a score_mod/mask_mod is being "
            "lowered; use where(cond, a, b) and the &, |, ~ operators instead of if/and/or/not"
        )

    def astype(self, dtype):
        return Sym(cast(self.e, _dtype_name(dtype)))

    # numpy interop: np.exp2(sym), np.where(sym, a, b) ...
    def __array_ufunc__(self, ufunc, method, *inputs, **kwargs):
        if method != "__call__" or kwargs:
            return NotImplemented
        fn = _NP_UFUNCS.get(ufunc.__name__)
        if fn is None:
            return NotImplemented
        return fn(*inputs)

    def __array_function__(self, func, types, args, kwargs):
        if func is np.where and not kwargs and len(args) == 3:
            return where(*args)
        return NotImplemented

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        name = getattr(func, "__name__", "")
        if name == "__getitem__" and len(args) == 2 and not isinstance(args[0], Sym):
            return _buffer_load(args[0], args[1])
        fn = _TORCH_FUNCS.get(name)
        if fn is None or kwargs:
            return NotImplemented
        return fn(*args)


def _dtype_name(dtype) -> str:
    if dtype in (bool, np.bool_) or str(dtype) in ("bool", "torch.bool"):
        return B1
    s = str(dtype)
    if "int" in s:
        return I32
    if "float" in s or dtype is float:
        return F32
    if dtype is int:
        return I32
    raise TypeError(f"unsupported dtype {dtype!r} in a mod trace")


# --------------------------------------------------------------------------------------
# function namespace usable on Sym / numpy / torch values alike
# --------------------------------------------------------------------------------------
def _any_sym(*xs) -> bool:
    return any(isinstance(x, Sym) for x in xs)


def _is_torch(*xs) -> bool:
    for x in xs:
        if type(x).__module__.startswith("torch"):
            return True
    return False


def _mk_unary(op, np_fn, torch_name):
    def f(x):
        if isinstance(x, Sym):
            return Sym(unary(op, x.e))
        if _is_torch(x):
            import torch

            return getattr(torch, torch_name)(x)
        return np_fn(x)

    f.__name__ = op
    return f


def _np_sigmoid(x):
    return 1.0 / (1.0 + np.exp(-np.asarray(x, dtype=np.float32)))


def _np_rsqrt(x):
    return 1.0 / np.sqrt(x)


exp = _mk_unary("exp", np.exp, "exp")
exp2 = _mk_unary("exp2", np.exp2, "exp2")
log = _mk_unary("log", np.log, "log")
log2 = _mk_unary("log2", np.log2, "log2")
sqrt = _mk_unary("sqrt", np.sqrt, "sqrt")
rsqrt = _mk_unary("rsqrt", _np_rsqrt, "rsqrt")
tanh = _mk_unary("tanh", np.tanh, "tanh")
sigmoid = _mk_unary("sigmoid", _np_sigmoid, "sigmoid")
sin = _mk_unary("sin", np.sin, "sin")
cos = _mk_unary("cos", np.cos, "cos")
floor = _mk_unary("floor", np.floor, "floor")
ceil = _mk_unary("ceil", np.ceil, "ceil")
isneginf = _mk_unary("isneginf", np.isneginf, "isneginf")
isinf = _mk_unary("isinf", np.isinf, "isinf")
isnan = _mk_unary("isnan", np.isnan, "isnan")
sign = _mk_unary("sign", np.sign, "sign")


def abs(x):  # noqa: A001 - mirrors jnp.abs
    if isinstance(x, Sym):
        return Sym(unary("abs", x.e))
    if _is_torch(x):
        import torch

        return torch.abs(x)
    return np.abs(x)


def where(c, a, b):
    if _any_sym(c, a, b):
        return Sym(select(_lift(c), _lift(a), _lift(b)))
    if _is_torch(c, a, b):
        import torch

        if not isinstance(c, torch.Tensor):
            c = torch.as_tensor(c)
        return torch.where(c, a, b)
    return np.where(c, a, b)


def _mk_binary(op, np_fn, torch_name):
    def f(a, b):
        if _any_sym(a, b):
            return Sym(binary(op, _lift(a), _lift(b)))
        if _is_torch(a, b):
            import torch

            if not isinstance(a, torch.Tensor):
                a = torch.as_tensor(a)
            if not isinstance(b, torch.Tensor):
                b = torch.as_tensor(b)
            return getattr(torch, torch_name)(a, b)
        return np_fn(a, b)

    f.__name__ = op
    return f


minimum = _mk_binary("min", np.minimum, "minimum")
maximum = _mk_binary("max", np.maximum, "maximum")
remainder = _mk_binary("rem", np.remainder, "remainder")
floor_divide = _mk_binary("floordiv", np.floor_divide, "floor_divide")
power = _mk_binary("pow", np.power, "pow")


def logical_and(a, b):
    if _any_sym(a, b):
        return Sym(binary("and", cast(_lift(a), B1), cast(_lift(b), B1)))
    if _is_torch(a, b):
        import torch

        return torch.logical_and(a, b)
    return np.logical_and(a, b)


def logical_or(a, b):
    if _any_sym(a, b):
        return Sym(binary("or", cast(_lift(a), B1), cast(_lift(b), B1)))
    if _is_torch(a, b):
        import torch

        return torch.logical_or(a, b)
    return np.logical_or(a, b)


def logical_not(a):
    if isinstance(a, Sym):
        return Sym(unary("not", cast(a.e, B1)))
    if _is_torch(a):
        import torch

        return torch.logical_not(a)
    return np.logical_not(a)


def ones(shape=(), dtype=np.float32):
    """Scalar one of the given dtype (the reference's combinators start from
    ``jnp.ones((), dtype=bool)``, flaxattention/core/blockmask.py:392)."""
    if shape not in ((), []):
        raise ValueError("only scalar constants can be created inside a mod")
    return np.ones((), dtype=np.bool_ if dtype in (bool, np.bool_) else dtype)[()]


def zeros(shape=(), dtype=np.float32):
    if shape not in ((), []):
        raise ValueError("only scalar constants can be created inside a mod")
    return np.zeros((), dtype=np.bool_ if dtype in (bool, np.bool_) else dtype)[()]


def float32(x):
    if isinstance(x, Sym):
        return x.astype(np.float32)
    if _is_torch(x):
        import torch

        return x.to(torch.float32)
    return np.float32(x)


def int32(x):
    if isinstance(x, Sym):
        return x.astype(np.int32)
    if _is_torch(x):
        import torch

        return x.to(torch.int32)
    return np.int32(x)


inf = float("inf")

_NP_UFUNCS = {
    "add": lambda a, b: Sym(binary("add", _lift(a), _lift(b))),
    "subtract": lambda a, b: Sym(binary("sub", _lift(a), _lift(b))),
    "multiply": lambda a, b: Sym(binary("mul", _lift(a), _lift(b))),
    "true_divide": lambda a, b: Sym(binary("div", _lift(a), _lift(b))),
    "divide": lambda a, b: Sym(binary("div", _lift(a), _lift(b))),
    "floor_divide": lambda a, b: Sym(binary("floordiv", _lift(a), _lift(b))),
    "remainder": lambda a, b: Sym(binary("rem", _lift(a), _lift(b))),
    "mod": lambda a, b: Sym(binary("rem", _lift(a), _lift(b))),
    "power": lambda a, b: Sym(binary("pow", _lift(a), _lift(b))),
    "minimum": minimum,
    "maximum": maximum,
    "less": lambda a, b: Sym(binary("lt", _lift(a), _lift(b))),
    "less_equal": lambda a, b: Sym(binary("le", _lift(a), _lift(b))),
    "greater": lambda a, b: Sym(binary("gt", _lift(a), _lift(b))),
    "greater_equal": lambda a, b: Sym(binary("ge", _lift(a), _lift(b))),
    "equal": lambda a, b: Sym(binary("eq", _lift(a), _lift(b))),
    "not_equal": lambda a, b: Sym(binary("ne", _lift(a), _lift(b))),
    "logical_and": logical_and,
    "logical_or": logical_or,
    "logical_not": logical_not,
    "bitwise_and": lambda a, b: Sym(binary("and", _lift(a), _lift(b))),
    "bitwise_or": lambda a, b: Sym(binary("or", _lift(a), _lift(b))),
    "bitwise_xor": lambda a, b: Sym(binary("xor", _lift(a), _lift(b))),
    "negative": lambda a: Sym(unary("neg", _lift(a))),
    "absolute": abs,
    "exp": exp, "exp2": exp2, "log": log, "log2": log2, "sqrt": sqrt, "tanh": tanh,
    "sin": sin, "cos": cos, "floor": floor, "ceil": ceil, "sign": sign,
    "isinf": isinf, "isnan": isnan,
}

_TORCH_FUNCS = {
    "where": where, "exp": exp, "exp2": exp2, "log": log, "log2": log2, "sqrt": sqrt,
    "rsqrt": rsqrt, "tanh": tanh, "sigmoid": sigmoid, "sin": sin, "cos": cos, "abs": abs,
    "floor": floor, "ceil": ceil, "minimum": minimum, "maximum": maximum,
    "remainder": remainder, "logical_and": logical_and, "logical_or": logical_or,
    "logical_not": logical_not, "isneginf": isneginf, "isinf": isinf, "isnan": isnan,
    "sign": sign, "pow": power,
}


# --------------------------------------------------------------------------------------
# tracing entry points
# --------------------------------------------------------------------------------------
def mod_arity(fn: Callable) -> int:
    """Number of parameters without a default: 5 marks a score_mod, 4 a mask_mod
    (flaxattention/core/common.py:20-39)."""
    return sum(
        1 for p in inspect.signature(fn).parameters.values() if p.default is inspect.Parameter.empty
    )


class TracedMod:
    """Result of tracing: ``kind`` is 'score' (float32 result) or 'mask' (bool result)."""

    def __init__(self, kind: str, root: Expr, buffers: Optional[List[object]] = None):
        self.kind = kind
        self.root = root
        self.buffers = buffers  # captured tensors the load nodes refer to (shared by a mod pair)

    @property
    def is_identity(self) -> bool:
        return self.kind == "score" and self.root.op == "score"

    @property
    def is_all_true(self) -> bool:
        return self.kind == "mask" and self.root.op == "const" and bool(self.root.value)

    def uses_score(self) -> bool:
        return _depends_on_score(self.root, {})


def _leaf_syms():
    return tuple(Sym(_B.leaf(n)) for n in _LEAVES)


def _traced(buffers: Optional[List[object]], run: Callable[[], Expr], kind: str) -> TracedMod:
    """Runs a trace with `buffers` as the registry that tensor[traced index] fills."""
    global _TRACE_BUFFERS
    bufs = [] if buffers is None else buffers
    prev, _TRACE_BUFFERS = _TRACE_BUFFERS, bufs
    try:
        root = run()
    finally:
        _TRACE_BUFFERS = prev
    return TracedMod(kind, root, bufs)


def trace_score_mod(fn: Callable, buffers: Optional[List[object]] = None) -> TracedMod:
    def run():
        s, b, h, q, kv = _leaf_syms()
        return cast(_lift(fn(s, b, h, q, kv)), F32)

    return _traced(buffers, run, "score")


def trace_mask_mod(fn: Callable, buffers: Optional[List[object]] = None) -> TracedMod:
    """Traces a mask_mod.  A 5-argument function is accepted as well and is then a
    score_mod evaluated on a zero score whose -inf results mark masked positions, the
    rule ``create_mask`` applies (flaxattention/core/blockmask.py:303-315)."""
    def run():
        s, b, h, q, kv = _leaf_syms()
        if mod_arity(fn) == 5:
            out = fn(Sym(_B.const(0.0, F32)), b, h, q, kv)
            return unary("not", unary("isneginf", cast(_lift(out), F32)))
        return cast(_lift(fn(b, h, q, kv)), B1)

    return _traced(buffers, run, "mask")


def _depends_on_score(e: Expr, memo) -> bool:
    r = memo.get(id(e))
    if r is None:
        r = e.op == "score" or any(_depends_on_score(a, memo) for a in e.args)
        memo[id(e)] = r
    return r


# --------------------------------------------------------------------------------------
# symbolic derivative with respect to the score
# --------------------------------------------------------------------------------------
def derivative(mod: TracedMod) -> TracedMod:
    if mod.kind != "score":
        raise ValueError("only a score_mod has a derivative")
    dep: Dict[int, bool] = {}
    memo: Dict[int, Expr] = {}
    zero, one = _B.const(0.0, F32), _B.const(1.0, F32)

    def d(e: Expr) -> Expr:
        if not _depends_on_score(e, dep):
            return zero
        got = memo.get(id(e))
        if got is not None:
            return got
        op, a = e.op, e.args
        if op == "score":
            r = one
        elif op == "add":
            r = binary("add", d(a[0]), d(a[1]))
        elif op == "sub":
            r = binary("sub", d(a[0]), d(a[1]))
        elif op == "neg":
            r = unary("neg", d(a[0]))
        elif op == "mul":
            r = binary("add", binary("mul", d(a[0]), a[1]), binary("mul", a[0], d(a[1])))
        elif op == "div":
            # (u/v)' = u'/v - u v'/v^2
            t1 = binary("div", d(a[0]), a[1])
            dv = d(a[1])
            if _is_const(dv, 0):
                r = t1
            else:
                r = binary("sub", t1, binary("div", binary("mul", a[0], dv), binary("mul", a[1], a[1])))
        elif op == "exp":
            r = binary("mul", e, d(a[0]))
        elif op == "exp2":
            r = binary("mul", binary("mul", e, _B.const(math.log(2.0), F32)), d(a[0]))
        elif op == "log":
            r = binary("div", d(a[0]), a[0])
        elif op == "log2":
            r = binary("div", d(a[0]), binary("mul", a[0], _B.const(math.log(2.0), F32)))
        elif op == "sqrt":
            r = binary("div", d(a[0]), binary("mul", _B.const(2.0, F32), e))
        elif op == "rsqrt":
            r = binary("mul", binary("mul", _B.const(-0.5, F32), binary("div", e, a[0])), d(a[0]))
        elif op == "tanh":
            r = binary("mul", binary("sub", one, binary("mul", e, e)), d(a[0]))
        elif op == "sigmoid":
            r = binary("mul", binary("mul", e, binary("sub", one, e)), d(a[0]))
        elif op == "sin":
            r = binary("mul", unary("cos", a[0]), d(a[0]))
        elif op == "cos":
            r = unary("neg", binary("mul", unary("sin", a[0]), d(a[0])))
        elif op == "erf":
            g = binary("mul", _B.const(2.0 / math.sqrt(math.pi), F32),
                       unary("exp", unary("neg", binary("mul", a[0], a[0]))))
            r = binary("mul", g, d(a[0]))
        elif op == "abs":
            r = binary("mul", unary("sign", a[0]), d(a[0]))
        elif op == "pow":
            if not _depends_on_score(a[1], dep):
                # u^c: c u^(c-1) u'
                r = binary("mul", binary("mul", a[1], binary("pow", a[0], binary("sub", a[1], one))), d(a[0]))
            else:
                # general: e * (v' ln u + v u'/u)
                r = binary("mul", e, binary("add", binary("mul", d(a[1]), unary("log", a[0])),
                                            binary("div", binary("mul", a[1], d(a[0])), a[0])))
        elif op == "min":
            r = select(binary("le", a[0], a[1]), d(a[0]), d(a[1]))
        elif op == "max":
            r = select(binary("ge", a[0], a[1]), d(a[0]), d(a[1]))
        elif op == "select":
            r = select(a[0], d(a[1]), d(a[2]))
        elif op == "rem":
            # float remainder u - floor(u / c) * c with a divisor that does not depend on the
            # score: piecewise u + const, so the derivative is u'; integer remainders are steps
            if e.dtype == F32 and not _depends_on_score(a[1], dep):
                r = d(a[0])
            else:
                r = zero
        elif op in ("floor", "ceil", "sign", "cast_i32", "cast_b1", "floordiv"):
            r = zero
        elif op == "cast_f32":
            r = zero  # the operand is an integer or bool: piecewise constant
        else:
            raise NotImplementedError(f"no derivative rule for '{op}'")
        memo[id(e)] = r
        return r

    return TracedMod("score", cast(d(mod.root), F32), mod.buffers)


# --------------------------------------------------------------------------------------
# affine decomposition:  score_mod(score, ...) == A(b,h,q,kv) * score + B(b,h,q,kv)
# --------------------------------------------------------------------------------------
def affine_parts(mod: TracedMod):
    """Returns (A, B) as index-only TracedMods when the score_mod is affine in the score
    (bias-type and scaling-type mods: ALiBi, relative biases, checkerboard ...), else None.
    Kernels use it to fold the softmax scale and the log2(e) factor into one FMA per score;
    A is also the derivative with respect to the score."""
    if mod.kind != "score":
        return None
    dep: Dict[int, bool] = {}
    memo: Dict[int, Optional[Tuple[Expr, Expr]]] = {}
    zero, one = _B.const(0.0, F32), _B.const(1.0, F32)
    fail = object()

    def go(e: Expr):
        if not _depends_on_score(e, dep):
            return (zero, cast(e, F32)) if e.dtype != B1 else None
        got = memo.get(id(e), fail)
        if got is not fail:
            return got
        op, a = e.op, e.args
        r = None
        if op == "score":
            r = (one, zero)
        elif op in ("add", "sub"):
            x, y = go(a[0]), go(a[1])
            if x and y:
                r = (binary(op, x[0], y[0]), binary(op, x[1], y[1]))
        elif op == "neg":
            x = go(a[0])
            if x:
                r = (unary("neg", x[0]), unary("neg", x[1]))
        elif op == "mul":
            for u, v in ((a[0], a[1]), (a[1], a[0])):
                if not _depends_on_score(v, dep):
                    x = go(u)
                    if x:
                        k = cast(v, F32)
                        r = (binary("mul", x[0], k), binary("mul", x[1], k))
                    break
        elif op == "div":
            if not _depends_on_score(a[1], dep):
                x = go(a[0])
                if x:
                    r = (binary("div", x[0], a[1]), binary("div", x[1], a[1]))
        elif op == "select":
            if not _depends_on_score(a[0], dep):
                x, y = go(a[1]), go(a[2])
                if x and y:
                    r = (select(a[0], x[0], y[0]), select(a[0], x[1], y[1]))
        memo[id(e)] = r
        return r

    res = go(mod.root)
    if res is None:
        return None
    return TracedMod("score", cast(res[0], F32), mod.buffers), TracedMod("score", cast(res[1], F32), mod.buffers)


# --------------------------------------------------------------------------------------
# index-linear biases:  B(b,h,q,kv) == B(.., x0) + (x - x0) * S(b,h,other index)   for x in {q, kv}
# --------------------------------------------------------------------------------------
def _depends_on(e: Expr, leaf: str, memo) -> bool:
    r = memo.get(id(e))
    if r is None:
        r = e.op == leaf or any(_depends_on(a, leaf, memo) for a in e.args)
        memo[id(e)] = r
    return r


def _int_bound(e: Expr, memo) -> float:
    """Upper bound of |value| of an integer expression made of indices (below 2^16 each), constants,
    +, - and *; infinity for anything else."""
    got = memo.get(id(e))
    if got is not None:
        return got
    if e.op in ("b", "h", "q", "kv"):
        r = float(1 << 16)
    elif e.op == "const" and e.dtype == I32:
        r = float(abs(int(e.value)))
    elif e.op in ("add", "sub") and e.dtype == I32:
        r = _int_bound(e.args[0], memo) + _int_bound(e.args[1], memo)
    elif e.op == "neg" and e.dtype == I32:
        r = _int_bound(e.args[0], memo)
    elif e.op == "mul" and e.dtype == I32:
        r = _int_bound(e.args[0], memo) * _int_bound(e.args[1], memo)
    else:
        r = float("inf")
    memo[id(e)] = r
    return r


def linear_slope(root: Expr, leaf: str) -> Optional[Expr]:
    """If the float expression ``root`` is linear in the index ``leaf`` ('q' or 'kv') - relative-position
    biases such as ALiBi are - returns its slope, an expression that does not read ``leaf``; else None.
    A kernel that walks along that index then evaluates the bias once per tile and adds multiples of
    the slope, instead of an integer subtraction, an int-to-float conversion (which shares the
    special-function unit with the exponentials) and a multiplication per element.
    Integer sub-expressions must stay below 2^24 in magnitude so that their conversion to float is
    exact term by term."""
    dep: Dict[int, bool] = {}
    bounds: Dict[int, float] = {}
    memo: Dict[int, object] = {}
    fail = object()

    def go(e: Expr):
        """slope of e (Expr of e's dtype, independent of leaf), or None when e is not linear in leaf"""
        if not _depends_on(e, leaf, dep):
            return _B.const(0, I32) if e.dtype == I32 else _B.const(0.0, F32)
        got = memo.get(id(e), fail)
        if got is not fail:
            return got
        op, a, r = e.op, e.args, None
        if e.dtype not in (I32, F32):
            r = None
        elif op == leaf:
            r = _B.const(1, I32)
        elif op in ("add", "sub"):
            x, y = go(a[0]), go(a[1])
            if x is not None and y is not None:
                r = binary(op, cast(x, e.dtype), cast(y, e.dtype))
        elif op == "neg":
            x = go(a[0])
            if x is not None:
                r = unary("neg", x)
        elif op == "mul":
            for u, v in ((a[0], a[1]), (a[1], a[0])):
                if not _depends_on(v, leaf, dep):
                    x = go(u)
                    if x is not None:
                        r = binary("mul", cast(x, e.dtype), v)
                    break
        elif op == "div" and e.dtype == F32:
            if not _depends_on(a[1], leaf, dep):
                x = go(a[0])
                if x is not None:
                    r = binary("div", cast(x, F32), a[1])
        elif op == "cast_f32" and a[0].dtype == I32:
            x = go(a[0])
            if x is not None and _int_bound(a[0], bounds) < float(1 << 24):
                r = cast(x, F32)
        memo[id(e)] = r
        return r

    res = go(root)
    if res is None:
        return None
    return cast(res, F32)


# --------------------------------------------------------------------------------------
# back ends
# --------------------------------------------------------------------------------------
def _topo(root: Expr) -> List[Expr]:
    order: List[Expr] = []
    seen = set()
    stack = [(root, False)]
    while stack:
        e, done = stack.pop()
        if done:
            order.append(e)
            continue
        if id(e) in seen:
            continue
        seen.add(id(e))
        stack.append((e, True))
        for a in reversed(e.args):
            if id(a) not in seen:
                stack.append((a, False))
    return order


import os as _os

_MAGIC_I2F = _os.environ.get("FLAXATTN_MAGIC_I2F", "0") == "1"
_IDX_BOUND = 1 << 21  # q, kv, b, h are taken to lie in [0, 2^21): sequences of up to 2M tokens


def _int_range(e: Expr, memo: Dict[int, Optional[Tuple[int, int]]]) -> Optional[Tuple[int, int]]:
    """Conservative value range of an int32 expression, or None when unknown."""
    got = memo.get(id(e), 0)
    if got != 0:
        return got
    r = None
    if e.dtype == I32:
        if e.op == "const":
            r = (e.value, e.value)
        elif e.op in ("q", "kv", "b", "h"):
            r = (0, _IDX_BOUND - 1)
        elif e.op in ("add", "sub"):
            a, b = _int_range(e.args[0], memo), _int_range(e.args[1], memo)
            if a and b:
                r = (a[0] + b[0], a[1] + b[1]) if e.op == "add" else (a[0] - b[1], a[1] - b[0])
        elif e.op == "neg":
            a = _int_range(e.args[0], memo)
            if a:
                r = (-a[1], -a[0])
        elif e.op == "and" and (_is_bit(e) or (e.args[1].op == "const" and e.args[1].value >= 0)):
            r = (0, 1) if _is_bit(e) else (0, e.args[1].value)
        elif e.op in ("xor", "or") and _is_bit(e):
            r = (0, 1)
        elif e.op == "cast_i32" and e.args[0].dtype == B1:
            r = (0, 1)
        elif e.op in ("min", "max"):
            a, b = _int_range(e.args[0], memo), _int_range(e.args[1], memo)
            if a and b:
                f = min if e.op == "min" else max
                r = (f(a[0], b[0]), f(a[1], b[1]))
        elif e.op == "abs":
            a = _int_range(e.args[0], memo)
            if a:
                r = (0, max(abs(a[0]), abs(a[1])))
    memo[id(e)] = r
    return r


_CTYPE = {I32: "int", F32: "float", B1: "bool"}


def _f32_literal(v: float) -> str:
    if math.isnan(v):
        return "__int_as_float(0x7fc00000)"
    if math.isinf(v):
        return "__int_as_float(0x7f800000)" if v > 0 else "__int_as_float(0xff800000)"
    return float(np.float32(v)).hex() + "f"


_CUDA_BIN = {
    "add": "({0} + {1})", "sub": "({0} - {1})", "mul": "({0} * {1})",
    "lt": "({0} < {1})", "le": "({0} <= {1})", "gt": "({0} > {1})", "ge": "({0} >= {1})",
    "eq": "({0} == {1})", "ne": "({0} != {1})",
}
_CUDA_UN_F = {
    "exp": "expf({0})", "exp2": "exp2f({0})", "log": "logf({0})", "log2": "log2f({0})",
    "sqrt": "sqrtf({0})", "rsqrt": "(1.0f / sqrtf({0}))", "tanh": "tanhf({0})",
    "sigmoid": "(1.0f / (1.0f + expf(-({0}))))", "sin": "sinf({0})", "cos": "cosf({0})",
    "floor": "floorf({0})", "ceil": "ceilf({0})", "erf": "erff({0})",
}


def to_cuda(mod: TracedMod, name: str) -> str:
    """Device function text.  Signature:
    ``float name(float score, int b, int h, int q, int kv)`` for a score mod (and its
    derivative), ``bool name(int b, int h, int q, int kv)`` for a mask mod."""
    lines: List[str] = []
    names: Dict[int, str] = {}
    ranges: Dict[int, Optional[Tuple[int, int]]] = {}
    n = 0
    for e in _topo(mod.root):
        if e.op in _LEAVES:
            names[id(e)] = e.op
            continue
        if e.op == "const":
            if e.dtype == F32:
                names[id(e)] = _f32_literal(e.value)
            elif e.dtype == I32:
                names[id(e)] = f"({e.value})" if e.value != -(1 << 31) else "(-2147483647 - 1)"
            else:
                names[id(e)] = "true" if e.value else "false"
            continue
        a = [names[id(x)] for x in e.args]
        t = e.dtype
        op = e.op
        if op in _CUDA_BIN:
            if t == I32 and op in ("add", "sub", "mul"):
                # wrap-around int32 arithmetic without signed-overflow UB
                sym = {"add": "+", "sub": "-", "mul": "*"}[op]
                rhs = f"(int)((unsigned){a[0]} {sym} (unsigned){a[1]})"
            else:
                rhs = _CUDA_BIN[op].format(*a)
        elif op == "div":
            rhs = f"({a[0]} / {a[1]})"
        elif op == "floordiv":
            rhs = f"fa_floordiv_i32({a[0]}, {a[1]})" if t == I32 else f"floorf({a[0]} / {a[1]})"
        elif op == "rem":
            rhs = f"fa_pymod_i32({a[0]}, {a[1]})" if t == I32 else f"fa_pymod_f32({a[0]}, {a[1]})"
        elif op == "pow":
            rhs = f"powf({a[0]}, {a[1]})"
        elif op == "min":
            rhs = f"min({a[0]}, {a[1]})" if t == I32 else f"fminf({a[0]}, {a[1]})"
        elif op == "max":
            rhs = f"max({a[0]}, {a[1]})" if t == I32 else f"fmaxf({a[0]}, {a[1]})"
        elif op == "and":
            rhs = f"({a[0]} && {a[1]})" if t == B1 else f"({a[0]} & {a[1]})"
        elif op == "or":
            rhs = f"({a[0]} || {a[1]})" if t == B1 else f"({a[0]} | {a[1]})"
        elif op == "xor":
            rhs = f"({a[0]} != {a[1]})" if t == B1 else f"({a[0]} ^ {a[1]})"
        elif op == "shl":
            rhs = f"(int)((unsigned){a[0]} << ({a[1]} & 31))"
        elif op == "shr":
            rhs = f"({a[0]} >> ({a[1]} & 31))"
        elif op == "neg":
            rhs = f"(-{a[0]})" if t == F32 else f"(int)(0u - (unsigned){a[0]})"
        elif op == "not":
            rhs = f"(!{a[0]})" if t == B1 else f"(~{a[0]})"
        elif op == "abs":
            rhs = f"fabsf({a[0]})" if t == F32 else f"abs({a[0]})"
        elif op == "sign":
            if t == F32:
                rhs = f"(({a[0]} > 0.0f) ? 1.0f : (({a[0]} < 0.0f) ? -1.0f : {a[0]}))"
            else:
                rhs = f"(({a[0]} > 0) - ({a[0]} < 0))"
        elif op == "isneginf":
            rhs = f"({a[0]} == __int_as_float(0xff800000))"
        elif op == "isinf":
            rhs = f"(fabsf({a[0]}) == __int_as_float(0x7f800000))"
        elif op == "isnan":
            rhs = f"({a[0]} != {a[0]})"
        elif op in _CUDA_UN_F:
            rhs = _CUDA_UN_F[op].format(*a)
        elif op == "select":
            rhs = f"({a[0]} ? {a[1]} : {a[2]})"
        elif op == "cast_f32":
            if e.args[0].dtype == I32:
                rg = _int_range(e.args[0], ranges)
                if _MAGIC_I2F and rg is not None and -(1 << 22) < rg[0] and rg[1] < (1 << 22):
                    # exact int -> float for |x| < 2^22 with an integer add and a float subtract
                    # (1.5 * 2^23 has the integer x in its low mantissa bits): keeps the
                    # conversion off the special-function unit the softmax exponentials need
                    rhs = f"(__int_as_float(0x4B400000 + {a[0]}) - 12582912.0f)"
                else:
                    rhs = f"(float)({a[0]})"
            else:
                rhs = f"({a[0]} ? 1.0f : 0.0f)"
        elif op == "cast_i32":
            rhs = f"(int)({a[0]})" if e.args[0].dtype == F32 else f"({a[0]} ? 1 : 0)"
        elif op == "cast_b1":
            rhs = f"({a[0]} != 0)" if e.args[0].dtype == I32 else f"({a[0]} != 0.0f)"
        elif op == "load":
            k, span, elem = e.value
            rhs = f"fa_ld_{elem}({k}, min(max({a[0]}, 0), {span - 1}))"
            if t == B1:
                rhs = f"({rhs} != 0)"
        else:
            raise NotImplementedError(op)
        var = f"t{n}"
        n += 1
        lines.append(f"  const {_CTYPE[t]} {var} = {rhs};")
        names[id(e)] = var
    ret = names[id(mod.root)]
    if mod.kind == "score":
        head = f"__device__ __forceinline__ float {name}(float score, int b, int h, int q, int kv) {{"
    else:
        head = f"__device__ __forceinline__ bool {name}(int b, int h, int q, int kv) {{"
    return "\n".join([head] + lines + [f"  return {ret};", "}"]) + "\n"


def _buffer_storage(buf, span: int) -> np.ndarray:
    """The first `span` elements of the storage behind a captured tensor (strided view undone)."""
    try:
        import torch

        if isinstance(buf, torch.Tensor):
            return torch.as_strided(buf.detach().cpu(), (span,), (1,)).numpy()
    except ImportError:  # pragma: no cover
        pass
    a = np.asarray(buf)
    return np.lib.stride_tricks.as_strided(a, (span,), (a.itemsize,))


def evaluate(mod: TracedMod, score, b, h, q, kv):
    """Numpy evaluation of the graph on broadcastable arrays (int32 indices, float32 score)."""
    env: Dict[int, np.ndarray] = {}
    leaves = {
        "score": None if score is None else np.asarray(score, dtype=np.float32),
        "b": np.asarray(b, dtype=np.int32), "h": np.asarray(h, dtype=np.int32),
        "q": np.asarray(q, dtype=np.int32), "kv": np.asarray(kv, dtype=np.int32),
    }
    npdt = {I32: np.int32, F32: np.float32, B1: np.bool_}
    with np.errstate(all="ignore"):
        for e in _topo(mod.root):
            op = e.op
            if op in _LEAVES:
                env[id(e)] = leaves[op]
                continue
            if op == "const":
                env[id(e)] = npdt[e.dtype](e.value)
                continue
            a = [env[id(x)] for x in e.args]
            t = npdt[e.dtype]
            if op == "add":
                r = a[0] + a[1]
            elif op == "sub":
                r = a[0] - a[1]
            elif op == "mul":
                r = a[0] * a[1]
            elif op == "div":
                r = np.float32(a[0]) / np.float32(a[1]) if np.ndim(a[0]) == 0 and np.ndim(a[1]) == 0 else a[0] / a[1]
            elif op == "floordiv":
                r = np.floor_divide(a[0], a[1])
            elif op == "rem":
                r = np.remainder(a[0], a[1])
            elif op == "pow":
                r = np.power(a[0], a[1])
            elif op == "min":
                r = np.minimum(a[0], a[1])
            elif op == "max":
                r = np.maximum(a[0], a[1])
            elif op == "and":
                r = np.logical_and(a[0], a[1]) if e.dtype == B1 else a[0] & a[1]
            elif op == "or":
                r = np.logical_or(a[0], a[1]) if e.dtype == B1 else a[0] | a[1]
            elif op == "xor":
                r = np.logical_xor(a[0], a[1]) if e.dtype == B1 else a[0] ^ a[1]
            elif op == "shl":
                r = a[0] << (a[1] & 31)
            elif op == "shr":
                r = a[0] >> (a[1] & 31)
            elif op in ("lt", "le", "gt", "ge", "eq", "ne"):
                r = {"lt": np.less, "le": np.less_equal, "gt": np.greater, "ge": np.greater_equal,
                     "eq": np.equal, "ne": np.not_equal}[op](a[0], a[1])
            elif op == "neg":
                r = -a[0]
            elif op == "not":
                r = np.logical_not(a[0]) if e.dtype == B1 else ~a[0]
            elif op == "abs":
                r = np.abs(a[0])
            elif op == "sign":
                r = np.sign(a[0])
            elif op == "isneginf":
                r = np.isneginf(a[0])
            elif op == "isinf":
                r = np.isinf(a[0])
            elif op == "isnan":
                r = np.isnan(a[0])
            elif op == "sigmoid":
                r = 1.0 / (1.0 + np.exp(-a[0]))
            elif op == "rsqrt":
                r = 1.0 / np.sqrt(a[0])
            elif op == "erf":
                from scipy.special import erf as _erf

                r = _erf(a[0])
            elif op in _UNARY_F:
                r = getattr(np, op)(a[0])
            elif op == "select":
                r = np.where(a[0], a[1], a[2])
            elif op.startswith("cast_"):
                r = a[0] != 0 if e.dtype == B1 else a[0]
            elif op == "load":
                k, span, _elem = e.value
                if mod.buffers is None:
                    raise ValueError("this mod reads captured buffers; evaluate a mod obtained from lower_mods")
                r = _buffer_storage(mod.buffers[k], span)[np.clip(np.asarray(a[0], dtype=np.int64), 0, span - 1)]
            else:
                raise NotImplementedError(op)
            env[id(e)] = np.asarray(r).astype(t, copy=False)
    return env[id(mod.root)]


_PRELUDE = r"""
__device__ __forceinline__ int fa_pymod_i32(int a, int b) {
  if (b == 0) return 0;
  if (b == -1) return 0;
  int r = a % b;
  return (r != 0 && ((r ^ b) < 0)) ? r + b : r;
}
__device__ __forceinline__ int fa_floordiv_i32(int a, int b) {
  if (b == 0) return 0;
  if (b == -1) return (int)(0u - (unsigned)a);
  int q = a / b;
  int r = a - q * b;
  return (r != 0 && ((r ^ b) < 0)) ? q - 1 : q;
}
__device__ __forceinline__ float fa_pymod_f32(float a, float b) {
  float r = fmodf(a, b);
  return (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) ? r + b : r;
}
"""


_BUFFER_PRELUDE = r"""
// Captured buffers: the host writes the device addresses here before every launch.
__constant__ const void* fa_mod_buf[FA_NUM_MOD_BUFS];
__device__ __forceinline__ int fa_ld_i32(int k, int i) { return __ldg((const int*)fa_mod_buf[k] + i); }
__device__ __forceinline__ int fa_ld_i64(int k, int i) { return (int)__ldg((const long long*)fa_mod_buf[k] + i); }
__device__ __forceinline__ int fa_ld_u8(int k, int i) { return (int)__ldg((const unsigned char*)fa_mod_buf[k] + i); }
__device__ __forceinline__ float fa_ld_f32(int k, int i) { return __ldg((const float*)fa_mod_buf[k] + i); }
"""


class ModSet:
    """The (score_mod, mask_mod) pair of one attention call, lowered.

    ``source`` is the device-code fragment: helper functions plus ``fa_score_mod``,
    ``fa_score_mod_grad`` and ``fa_mask_mod`` together with the ``FA_HAS_*`` macros the
    kernel templates test.  ``key`` is a SHA-256 of that text, used as the cache key of
    compiled kernels and of this object.
    """

    def __init__(self, score: Optional[TracedMod], mask: Optional[TracedMod], buffers: Optional[List[object]] = None):
        self.score = score if (score is not None and not score.is_identity) else None
        self.mask = mask if (mask is not None and not mask.is_all_true) else None
        # tensors the mods close over and index (document ids, learned biases ...); the load
        # nodes of both mods number them in this list
        self.buffers: List[object] = list(buffers) if buffers else []
        parts = [_PRELUDE]
        if self.buffers:
            parts.append(f"#define FA_NUM_MOD_BUFS {len(self.buffers)}\n")
            parts.append(_BUFFER_PRELUDE)
        parts.append(f"#define FA_HAS_SCORE_MOD {1 if self.score is not None else 0}\n")
        parts.append(f"#define FA_HAS_MASK_MOD {1 if self.mask is not None else 0}\n")
        self.affine = None
        if self.score is not None:
            self.grad = derivative(self.score)
            parts.append(to_cuda(self.score, "fa_score_mod"))
            parts.append(to_cuda(self.grad, "fa_score_mod_grad"))
            self.affine = affine_parts(self.score)
            if self.affine is not None:
                # score_mod(s) == fa_score_mul(...) * s + fa_score_add(...); both ignore `score`
                parts.append("#define FA_SCORE_AFFINE 1\n")
                n_ops = sum(1 for t in self.affine for e in _topo(t.root) if e.args)
                if n_ops <= 10:
                    # cheap enough to evaluate twice (row maximum pass and exponent pass) instead of
                    # writing the modified scores back between the passes
                    parts.append("#define FA_SCORE_AFFINE_CHEAP 1\n")
                parts.append(to_cuda(self.affine[0], "fa_score_mul"))
                parts.append(to_cuda(self.affine[1], "fa_score_add"))
                # B already multiplied by log2(e), with the constant folded into row-invariant factors
                b2 = TracedMod("score", binary("mul", self.affine[1].root, _B.const(math.log2(math.e), F32)), self.affine[1].buffers)
                parts.append(to_cuda(b2, "fa_score_add2"))
                # A bias that is linear in kv (q) under a multiplier that does not read kv (q): the kernels
                # take the bias at the first column of a chunk and add multiples of the slope
                self.linear = {}
                for leaf, tag in (("kv", "KV"), ("q", "Q")):
                    slope = linear_slope(b2.root, leaf)
                    if slope is not None and not _depends_on(self.affine[0].root, leaf, {}):
                        self.linear[leaf] = slope
                        parts.append(f"#define FA_SCORE_LINEAR_{tag} 1\n")
                        parts.append(to_cuda(TracedMod("score", slope, b2.buffers), f"fa_score_add2_d{leaf}"))
        else:
            self.grad = None
            parts.append(
                "__device__ __forceinline__ float fa_score_mod(float score, int, int, int, int) { return score; }\n"
                "__device__ __forceinline__ float fa_score_mod_grad(float, int, int, int, int) { return 1.0f; }\n"
            )
        if self.mask is not None:
            parts.append(to_cuda(self.mask, "fa_mask_mod"))
        else:
            parts.append("__device__ __forceinline__ bool fa_mask_mod(int, int, int, int) { return true; }\n")
        self.source = "".join(parts)
        self.key = hashlib.sha256(self.source.encode()).hexdigest()


def _trace_any(fn: Callable, kind: str, bufs: List[object]) -> TracedMod:
    """Symbolic call first; a mod written with jax.numpy rejects the symbols and is traced through
    its jaxpr instead (jax_frontend), when JAX is installed."""
    try:
        return trace_score_mod(fn, bufs) if kind == "score" else trace_mask_mod(fn, bufs)
    except Exception as first:
        try:
            import jax  # noqa: F401
        except ImportError:
            raise first from None
        from .jax_frontend import trace_with_jax

        try:
            return trace_with_jax(fn, kind)
        except Exception:
            raise first from None


_MODSET_CACHE: Dict[Tuple[Optional[int], Optional[int]], Tuple[object, object, ModSet]] = {}


def lower_mods(score_mod: Optional[Callable], mask_mod: Optional[Callable]) -> ModSet:
    """Traces and lowers a pair of mods; cached on the identity of the callables (the
    reference keys its jit cache the same way: mods are static arguments,
    flaxattention/core/attention.py:169)."""
    k = (None if score_mod is None else id(score_mod), None if mask_mod is None else id(mask_mod))
    hit = _MODSET_CACHE.get(k)
    if hit is not None and hit[0] is score_mod and hit[1] is mask_mod:
        return hit[2]
    bufs: List[object] = []
    s = _trace_any(score_mod, "score", bufs) if score_mod is not None else None
    m = _trace_any(mask_mod, "mask", bufs) if mask_mod is not None else None
    ms = ModSet(s, m, bufs)
    if len(_MODSET_CACHE) > 4096:
        _MODSET_CACHE.clear()
    _MODSET_CACHE[k] = (score_mod, mask_mod, ms)
    return ms
