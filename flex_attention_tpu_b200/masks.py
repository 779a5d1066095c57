"""Mask factories with the reference's names and signatures (reference ``masks.py``).

Each factory returns ``(mask_fn, block_mask_fn)`` exactly like the reference: ``mask_fn(q_idx, k_idx)``
gives the element-wise keep matrix and ``block_mask_fn(q_block, k_block)`` says whether a tile pair holds
any kept pair.  Both remain ordinary callables on NumPy / torch index arrays (so they can be compared with
the oracle), and both carry a ``.spec`` tag.  The CUDA entry points never call them: they read the tag and
select the compile-time mask functor and the mask-map classification in the library.  An untagged callable
cannot be run on the GPU and is rejected with ``NotImplementedError``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class MaskSpec:
    kind: str                                   # none | causal | sliding_window | sliding_window_causal | document | s2
    window: int = 0
    stride: int = 0
    doc_lengths: Optional[Tuple[int, ...]] = None   # static document layout shared by all batch rows
    block_q: int = 128
    block_k: int = 128


class _Tagged:
    def __init__(self, fn, spec):
        self._fn, self.spec = fn, spec
        self.__name__ = getattr(fn, "__name__", "mask_fn")

    def __call__(self, *a, **kw):
        return self._fn(*a, **kw)


def _pair(mask_fn, block_fn, spec):
    return _Tagged(mask_fn, spec), _Tagged(block_fn, spec)


def _col(x):
    return x[:, None]


def _row(x):
    return x[None, :]


def place_holder(block_q, block_k_major):
    """No mask (reference masks.py:3-6)."""
    spec = MaskSpec("none", block_q=block_q, block_k=block_k_major)

    def p(q_block_idx, k_block_idx):
        return True
    return _pair(p, p, spec)


def make_causal_mask_fns(block_q, block_k_major):
    """Keep q >= k (reference masks.py:8-30)."""
    spec = MaskSpec("causal", block_q=block_q, block_k=block_k_major)

    def causal_mask_fn(q_idx, k_idx):
        return _col(q_idx) >= _row(k_idx)

    def causal_block_mask_fn(q_block_idx, k_block_idx):
        return k_block_idx * block_k_major <= (q_block_idx + 1) * block_q - 1
    return _pair(causal_mask_fn, causal_block_mask_fn, spec)


def make_sliding_window_mask_fns(block_q, block_k, window_size, causal=False):
    """Keep q - k < window (reference masks.py:33-83; like the reference this is NOT causal unless
    ``causal=True`` is passed, an extension that also requires q >= k)."""
    spec = MaskSpec("sliding_window_causal" if causal else "sliding_window", window=int(window_size),
                    block_q=block_q, block_k=block_k)

    def sliding_window_mask_fn(q_idx, k_idx):
        dist = _col(q_idx) - _row(k_idx)
        keep = dist < window_size
        return keep & (dist >= 0) if causal else keep

    def sliding_window_block_mask_fn(q_block_idx, k_block_idx):
        q_start, q_end = q_block_idx * block_q, (q_block_idx + 1) * block_q - 1
        k_start, k_end = k_block_idx * block_k, (k_block_idx + 1) * block_k - 1
        keep = (q_start - k_end) < window_size
        return keep & (k_start <= q_end) if causal else keep
    return _pair(sliding_window_mask_fn, sliding_window_block_mask_fn, spec)


def make_jagged_mask_fns(block_q, block_k, doc_lengths: Sequence[int]):
    """Document mask: same document and causal (reference masks.py:88-141).  ``doc_lengths`` is one static
    layout shared by every batch row, as in the reference; per-row layouts go through ``segment_ids``."""
    lengths = tuple(int(x) for x in doc_lengths)
    boundaries = np.cumsum((0,) + lengths)
    spec = MaskSpec("document", doc_lengths=lengths, block_q=block_q, block_k=block_k)

    def get_doc_id(idx):
        return np.searchsorted(boundaries[1:], np.asarray(idx), side="right")

    def jagged_mask_fn(q_idx, k_idx):
        q_idx, k_idx = np.asarray(q_idx), np.asarray(k_idx)
        return (_col(get_doc_id(q_idx)) == _row(get_doc_id(k_idx))) & (_col(q_idx) >= _row(k_idx))

    def jagged_block_mask_fn(q_b, k_b):
        q_start, q_end = q_b * block_q, (q_b + 1) * block_q - 1
        k_start, k_end = k_b * block_k, (k_b + 1) * block_k - 1
        lo = np.maximum(get_doc_id(q_start), get_doc_id(k_start))
        hi = np.minimum(get_doc_id(q_end), get_doc_id(k_end))
        return (lo <= hi) & (k_start <= q_end)
    return _pair(jagged_mask_fn, jagged_block_mask_fn, spec)


def make_s2_mask_fns(block_q, block_k, window_size, stride):
    """S2 attention: causal window OR causal strided keys (reference masks.py:143-179)."""
    spec = MaskSpec("s2", window=int(window_size), stride=int(stride), block_q=block_q, block_k=block_k)

    def s2_mask_fn(q_idx, k_idx):
        dist = _col(q_idx) - _row(k_idx)
        is_local = (dist >= 0) & (dist < window_size)
        return is_local | (_row(k_idx % stride == 0) & (dist >= 0))

    def s2_block_mask_fn(q_b, k_b):
        # like the reference, assumes block_k >= stride so that every key block holds a strided key
        return k_b * block_k <= (q_b + 1) * block_q - 1
    return _pair(s2_mask_fn, s2_block_mask_fn, spec)


def doc_ids_from_lengths(doc_lengths: Sequence[int]) -> np.ndarray:
    """[S] int32 document id of every position for a list of document lengths."""
    return np.repeat(np.arange(len(doc_lengths), dtype=np.int32), np.asarray(doc_lengths, dtype=np.int64))


def spec_of(mask_fn, block_mask_fn=None) -> Optional[MaskSpec]:
    """MaskSpec carried by a (mask_fn, block_mask_fn) pair; None if both are None."""
    for fn in (mask_fn, block_mask_fn):
        if fn is not None:
            spec = getattr(fn, "spec", None)
            if spec is None:
                raise NotImplementedError(
                    "mask callables must come from the factories in this module: arbitrary Python mask "
                    "functions cannot be compiled into the CUDA kernels")
            return spec
    return None
