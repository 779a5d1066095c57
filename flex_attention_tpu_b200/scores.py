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
    kind: str                                 # none | alibi | softcap
    cap: float = 0.0
    slopes: Optional[Tuple[float, ...]] = None    # one per head, or a single value for every head


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


def alibi_slopes(num_heads: int) -> np.ndarray:
    """The standard ALiBi schedule slope_h = 2^(-8 (h+1) / H)."""
    return np.exp2(-8.0 * np.arange(1, num_heads + 1) / num_heads).astype(np.float32)


def spec_of(score_fn) -> Optional[ScoreSpec]:
    if score_fn is None:
        return None
    spec = getattr(score_fn, "spec", None)
    if spec is None:
        raise NotImplementedError(
            "score_fn must come from the factories in this module (or pass through make_jax_score_fn "
            "with its tag intact): arbitrary Python score functions cannot be compiled into the CUDA kernels")
    return spec
