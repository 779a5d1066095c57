"""Symbolic tracing of a user score function into CUDA source, with its derivative.

The reference turns a user's Python score function into fusable JAX by rewriting its AST (``util.py:22-189``,
``ToJaxTransformer`` / ``make_jax_score_fn``) and differentiates it with ``jax.vjp`` inside the backward kernels
(``flex_attention_dq_bwd.py:340-345,373-380``).  Here the same two jobs are done by tracing: the function is
called once with symbolic arguments, every arithmetic operation it performs builds a node of a small expression
tree, and the tree is then (a) printed as a CUDA C++ expression, (b) differentiated symbolically with respect to
the score and printed again, (c) evaluated on NumPy arrays, which is what the CPU oracle uses for the same
function.  The two CUDA expressions are compiled into the attention kernels at run time by the library
(``flexattn_user_score_create``).

A score function may be written in either of two forms:

    f(score, b, h, q_idx, k_idx)     the scaled score s = sm_scale * <q_i, k_j> plus batch, head and positions
    f(q_tile, k_tile)                the reference's form; ``q_tile @ k_tile.T`` (or ``np.dot(q_tile, k_tile.T)``)
                                     yields the scaled score, nothing else may be done with the tiles

using Python arithmetic (+ - * / and unary -, ** with a constant exponent), comparisons with ``where``, and the
functions of this module or their NumPy namesakes (``np.tanh(x)`` works on a traced value): tanh, exp, log,
sqrt, abs, sigmoid, minimum, maximum, where.
"""
from __future__ import annotations

import inspect
import math
from typing import Callable, Dict, Tuple, Union

import numpy as np

Number = Union[int, float]


class Expr:
    """A node: op in {const, var, add, sub, mul, div, neg, tanh, exp, log, sqrt, abs, min, max, ge, gt, where}."""
    __slots__ = ("op", "args", "value")
    __array_priority__ = 1000

    def __init__(self, op, args=(), value=None):
        self.op, self.args, self.value = op, tuple(args), value

    # ---- construction
    @staticmethod
    def wrap(x) -> "Expr":
        if isinstance(x, Expr):
            return x
        if isinstance(x, (int, float, np.integer, np.floating)):
            return Expr("const", value=float(x))
        raise TypeError(f"cannot use {type(x).__name__} inside a score function: only numbers and traced values")

    def __add__(self, o): return _fold("add", self, Expr.wrap(o))
    def __radd__(self, o): return _fold("add", Expr.wrap(o), self)
    def __sub__(self, o): return _fold("sub", self, Expr.wrap(o))
    def __rsub__(self, o): return _fold("sub", Expr.wrap(o), self)
    def __mul__(self, o): return _fold("mul", self, Expr.wrap(o))
    def __rmul__(self, o): return _fold("mul", Expr.wrap(o), self)
    def __truediv__(self, o): return _fold("div", self, Expr.wrap(o))
    def __rtruediv__(self, o): return _fold("div", Expr.wrap(o), self)
    def __neg__(self): return _fold("neg", self)
    def __pos__(self): return self
    def __abs__(self): return Expr("abs", (self,))
    def __ge__(self, o): return Expr("ge", (self, Expr.wrap(o)))
    def __gt__(self, o): return Expr("gt", (self, Expr.wrap(o)))
    def __le__(self, o): return Expr("ge", (Expr.wrap(o), self))
    def __lt__(self, o): return Expr("gt", (Expr.wrap(o), self))

    def __pow__(self, n):
        if not isinstance(n, (int, np.integer)) or not 0 <= int(n) <= 8:
            raise TypeError("** in a score function needs a constant integer exponent between 0 and 8")
        out = Expr.wrap(1.0)
        for _ in range(int(n)):
            out = out * self
        return out

    def __bool__(self):
        raise TypeError("a traced value has no truth value: use where(cond, a, b) instead of if / and / or")

    # NumPy functions applied to a traced value (np.tanh(x), np.maximum(x, 0.0) ...) build nodes too
    def __array_ufunc__(self, ufunc, method, *inputs, **kwargs):
        if method != "__call__" or kwargs:
            return NotImplemented
        table = {np.add: lambda a, b: a + b, np.subtract: lambda a, b: a - b, np.multiply: lambda a, b: a * b,
                 np.true_divide: lambda a, b: a / b, np.negative: lambda a: -a, np.tanh: tanh, np.exp: exp,
                 np.log: log, np.sqrt: sqrt, np.absolute: lambda a: abs(a), np.minimum: minimum, np.maximum: maximum,
                 np.greater_equal: lambda a, b: a >= b, np.greater: lambda a, b: a > b,
                 np.less_equal: lambda a, b: a <= b, np.less: lambda a, b: a < b}
        fn = table.get(ufunc)
        if fn is None:
            return NotImplemented
        return fn(*[Expr.wrap(x) for x in inputs])


def _fold(op, *args) -> Expr:
    """Node construction with the few simplifications that keep derivatives readable (x*1, x+0, 0*x, constants)."""
    if all(a.op == "const" for a in args):
        v = [a.value for a in args]
        return Expr("const", value={"add": lambda: v[0] + v[1], "sub": lambda: v[0] - v[1], "mul": lambda: v[0] * v[1],
                                    "div": lambda: v[0] / v[1], "neg": lambda: -v[0]}[op]())
    is_c = lambda a, val: a.op == "const" and a.value == val
    if op == "add":
        if is_c(args[0], 0.0): return args[1]
        if is_c(args[1], 0.0): return args[0]
    if op == "sub" and is_c(args[1], 0.0):
        return args[0]
    if op == "mul":
        if is_c(args[0], 0.0) or is_c(args[1], 0.0): return Expr("const", value=0.0)
        if is_c(args[0], 1.0): return args[1]
        if is_c(args[1], 1.0): return args[0]
    if op == "div" and is_c(args[1], 1.0):
        return args[0]
    if op == "neg" and args[0].op == "neg":
        return args[0].args[0]
    return Expr(op, args)


def tanh(x): return Expr("tanh", (Expr.wrap(x),))
def exp(x): return Expr("exp", (Expr.wrap(x),))
def log(x): return Expr("log", (Expr.wrap(x),))
def sqrt(x): return Expr("sqrt", (Expr.wrap(x),))
def minimum(a, b): return Expr("min", (Expr.wrap(a), Expr.wrap(b)))
def maximum(a, b): return Expr("max", (Expr.wrap(a), Expr.wrap(b)))
def where(c, a, b): return Expr("where", (Expr.wrap(c), Expr.wrap(a), Expr.wrap(b)))
def sigmoid(x): return 1.0 / (1.0 + exp(-Expr.wrap(x)))


VARS = ("s", "b", "h", "q_idx", "k_idx")
_CUDA_VAR = {"s": "s", "b": "(float)b", "h": "(float)h", "q_idx": "(float)i", "k_idx": "(float)j"}


def _const_literal(v: float) -> str:
    if math.isinf(v) or math.isnan(v):
        raise ValueError("score functions may not contain infinities or NaNs")
    return repr(float(np.float32(v))) + "f"


def to_cuda(e: Expr) -> str:
    """The tree as a CUDA C++ float expression in s (float) and b, h, i, j (int)."""
    a = [to_cuda(x) for x in e.args]
    if e.op == "const": return _const_literal(e.value)
    if e.op == "var": return _CUDA_VAR[e.value]
    if e.op == "add": return f"({a[0]} + {a[1]})"
    if e.op == "sub": return f"({a[0]} - {a[1]})"
    if e.op == "mul": return f"({a[0]} * {a[1]})"
    if e.op == "div": return f"({a[0]} / {a[1]})"
    if e.op == "neg": return f"(-{a[0]})"
    if e.op == "tanh": return f"tanhf({a[0]})"
    if e.op == "exp": return f"expf({a[0]})"
    if e.op == "log": return f"logf({a[0]})"
    if e.op == "sqrt": return f"sqrtf({a[0]})"
    if e.op == "abs": return f"fabsf({a[0]})"
    if e.op == "min": return f"fminf({a[0]}, {a[1]})"
    if e.op == "max": return f"fmaxf({a[0]}, {a[1]})"
    if e.op == "ge": return f"({a[0]} >= {a[1]})"
    if e.op == "gt": return f"({a[0]} > {a[1]})"
    if e.op == "where": return f"({a[0]} ? {a[1]} : {a[2]})"
    raise ValueError(e.op)


def evaluate(e: Expr, env: Dict[str, np.ndarray]) -> np.ndarray:
    """The tree on NumPy arrays (float32 arithmetic), broadcasting the variables of `env`."""
    f32 = np.float32
    a = [evaluate(x, env) for x in e.args]
    if e.op == "const": return f32(e.value)
    if e.op == "var": return np.asarray(env[e.value], dtype=f32)
    if e.op == "add": return a[0] + a[1]
    if e.op == "sub": return a[0] - a[1]
    if e.op == "mul": return a[0] * a[1]
    if e.op == "div": return a[0] / a[1]
    if e.op == "neg": return -a[0]
    if e.op == "tanh": return np.tanh(a[0])
    if e.op == "exp": return np.exp(a[0])
    if e.op == "log": return np.log(a[0])
    if e.op == "sqrt": return np.sqrt(a[0])
    if e.op == "abs": return np.abs(a[0])
    if e.op == "min": return np.minimum(a[0], a[1])
    if e.op == "max": return np.maximum(a[0], a[1])
    if e.op == "ge": return a[0] >= a[1]
    if e.op == "gt": return a[0] > a[1]
    if e.op == "where": return np.where(a[0], a[1], a[2]).astype(f32)
    raise ValueError(e.op)


def diff(e: Expr) -> Expr:
    """d e / d s, symbolically."""
    c = lambda v: Expr("const", value=float(v))
    if e.op == "const": return c(0.0)
    if e.op == "var": return c(1.0 if e.value == "s" else 0.0)
    a = e.args
    if e.op == "add": return diff(a[0]) + diff(a[1])
    if e.op == "sub": return diff(a[0]) - diff(a[1])
    if e.op == "mul": return diff(a[0]) * a[1] + a[0] * diff(a[1])
    if e.op == "div": return diff(a[0]) / a[1] - (a[0] * diff(a[1])) / (a[1] * a[1])
    if e.op == "neg": return -diff(a[0])
    if e.op == "tanh": return (1.0 - e * e) * diff(a[0])
    if e.op == "exp": return e * diff(a[0])
    if e.op == "log": return diff(a[0]) / a[0]
    if e.op == "sqrt": return diff(a[0]) / (2.0 * e)
    if e.op == "abs": return where(a[0] >= 0.0, diff(a[0]), -diff(a[0]))
    if e.op == "min": return where(a[1] >= a[0], diff(a[0]), diff(a[1]))
    if e.op == "max": return where(a[0] >= a[1], diff(a[0]), diff(a[1]))
    if e.op == "where": return where(a[0], diff(a[1]), diff(a[2]))
    if e.op in ("ge", "gt"):
        raise TypeError("a comparison can only be used as the condition of where()")
    raise ValueError(e.op)


class _Tile:
    """Stand-in for a q / k tile of the reference's two-argument form: only q @ k.T (= the scaled score) is allowed."""
    def __init__(self, name, transposed=False):
        self.name, self.transposed = name, transposed

    @property
    def T(self):
        return _Tile(self.name, not self.transposed)

    def transpose(self, *a):
        return self.T

    def __matmul__(self, other):
        if isinstance(other, _Tile) and self.name == "q" and other.name == "k" and not self.transposed and other.transposed:
            return Expr("var", value="s")
        raise TypeError("the only tile operation a score function may do is q_tile @ k_tile.T")

    def dot(self, other):
        return self.__matmul__(other)

    def __array_function__(self, func, types, args, kwargs):
        if func in (np.dot, np.matmul) and len(args) == 2:
            return args[0].__matmul__(args[1])
        if func is np.transpose:
            return args[0].T
        return NotImplemented


def trace(fn: Union[Callable, str]) -> Tuple[Expr, Expr]:
    """(score expression, d score / d s) of a user score function (see the module docstring for the accepted
    forms) or of a Python expression string in s, b, h, q_idx, k_idx.  Raises TypeError when the function does
    something that cannot be traced."""
    sym = {v: Expr("var", value=v) for v in VARS}
    if isinstance(fn, str):
        ns = dict(sym, tanh=tanh, exp=exp, log=log, sqrt=sqrt, abs=abs, sigmoid=sigmoid, minimum=minimum,
                  maximum=maximum, where=where, np=np, score=sym["s"])
        out = eval(fn, {"__builtins__": {}}, ns)       # noqa: S307 - an expression over the symbols above only
    else:
        n = len([p for p in inspect.signature(fn).parameters.values()
                 if p.default is inspect.Parameter.empty and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)])
        if n == 2:
            out = fn(_Tile("q"), _Tile("k"))
        elif n == 5:
            out = fn(*[sym[v] for v in VARS])
        else:
            raise TypeError("a score function takes (score, b, h, q_idx, k_idx) or (q_tile, k_tile)")
    out = Expr.wrap(out)
    return out, diff(out)
