"""score_mod factories with the reference's names (reference ``scores.py``).

The returned callables still compute ``score_fn(q_tile, k_tile) -> [Bq, Bk]`` on NumPy / torch arrays, and
carry a ``.spec`` tag the CUDA entry points read to pick the compile-time score functor.

Convention of this build: the functor acts on the scaled score ``s = sm_scale * q.k``; ALiBi is real ALiBi
(global distance, one slope per head, bias = -slope_h * (i - j)) instead of the reference's tile-local demo
(scores.py:3-11).  With ``sm_scale == 1`` and a single tile the two coincide for i >= j.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np


@dataclass(frozen=True)
class ScoreSpec:
    kind: str                                 # none | alibi | softcap | user
    cap: float = 0.0
    slopes: Optional[Tuple[float, ...]] = None    # one per head, or a single value for every head
    expr: Optional[str] = None                # user: CUDA expression of the score function t = f(s, b, h, i, j)
    dexpr: Optional[str] = None               # user: CUDA expression of df / ds


class _Tagged:
    def __init__(self, fn, spec):
        self._fn, self.spec = fn, spec
        self.__name__ = getattr(fn, "__name__", "score_fn")

    def __call__(self, *a, **kw):
        return self._fn(*a, **kw)


def make_alibi_score_fn(slope=0.5):
    """Linear distance penalty.  ``slope`` is a scalar (all heads) or a sequence with one slope per head."""
    slopes = tuple(float(s) for s in np.atleast_1d(np.asarray(slope, dtype=np.float64)))

    def alibi_score(q_tile, k_tile, head=0):
        m, n = q_tile.shape[0], k_tile.shape[0]
        dist = np.arange(m)[:, None] - np.arange(n)[None, :]
        return q_tile @ k_tile.T - slopes[head % len(slopes)] * dist
    return _Tagged(alibi_score, ScoreSpec("alibi", slopes=slopes))


def make_softcap_score_fn(cap=30.0):
    """Gemma-2 style soft cap: cap * tanh(score / cap) (reference scores.py:13-18)."""
    cap = float(cap)

    def softcap_score(q_tile, k_tile):
        return cap * np.tanh((q_tile @ k_tile.T) / cap)
    return _Tagged(softcap_score, ScoreSpec("softcap", cap=cap))


def make_user_score_fn(fn):
    """Any score function the tracer of ``score_expr`` can follow, compiled into the tensor-core kernels at run time.

    ``fn`` is ``f(score, b, h, q_idx, k_idx)`` on the scaled score, the reference's ``f(q_tile, k_tile)`` whose only
    tile operation is ``q_tile @ k_tile.T``, or a Python expression string over ``s, b, h, q_idx, k_idx``.  The
    counterpart of the reference's ``make_jax_score_fn`` (``util.py:150-189``): there the function's AST is rewritten
    into JAX and ``jax.vjp`` differentiates it; here it is traced into a CUDA expression and differentiated
    symbolically.  The returned callable evaluates the same expression tree on NumPy arrays:
    ``score_fn(s, b, h, q_idx, k_idx)`` and ``score_fn.dscore(...)``, which is what a CPU check needs.  bfloat16
    inputs with head_dim 64 or 128 only."""
    from . import score_expr as se
    e, d = se.trace(fn)

    def user_score(s, b=0, h=0, q_idx=0, k_idx=0):
        return se.evaluate(e, dict(s=s, b=b, h=h, q_idx=q_idx, k_idx=k_idx))

    tagged = _Tagged(user_score, ScoreSpec("user", expr=se.to_cuda(e), dexpr=se.to_cuda(d)))
    tagged.dscore = lambda s, b=0, h=0, q_idx=0, k_idx=0: se.evaluate(d, dict(s=s, b=b, h=h, q_idx=q_idx, k_idx=k_idx))
    return tagged


def alibi_slopes(num_heads: int) -> np.ndarray:
    """The standard ALiBi schedule slope_h = 2^(-8 (h+1) / H)."""
    return np.exp2(-8.0 * np.arange(1, num_heads + 1) / num_heads).astype(np.float32)


def spec_of(score_fn) -> Optional[ScoreSpec]:
    if score_fn is None:
        return None
    spec = getattr(score_fn, "spec", None)
    if spec is None:
        raise NotImplementedError(
            "score_fn must come from the factories in this module or from util.make_jax_score_fn / "
            "scores.make_user_score_fn, which trace a Python score function into the CUDA kernels: an untraced "
            "Python callable cannot run on the GPU")
    return spec
