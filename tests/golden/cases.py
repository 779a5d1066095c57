"""Definitions of the golden cases: shared by ``make_golden.py`` (which runs the reference's
sources on them) and by the tests (which rebuild the same inputs from the seeds)."""
from __future__ import annotations

import numpy as np

_INV = lambda d: float(1.0 / np.sqrt(d))

# name -> shape [B,H,Sq,Sk,D], seed, mask / score description in the reference oracle's vocabulary
CASES = {
    "dense":         dict(shape=(1, 2, 96, 96, 32), seed=11, sm_scale=_INV(32)),
    "causal":        dict(shape=(1, 2, 96, 96, 32), seed=12, sm_scale=_INV(32), causal=True),
    "window_causal": dict(shape=(1, 2, 96, 96, 32), seed=13, sm_scale=_INV(32), causal=True, window=24),
    "window":        dict(shape=(1, 2, 96, 96, 32), seed=14, sm_scale=_INV(32), window=24),
    "document":      dict(shape=(2, 2, 96, 96, 32), seed=15, sm_scale=_INV(32), causal=True,
                          docs=[[30, 40, 26], [7, 50, 39]]),
    "s2":            dict(shape=(1, 2, 96, 96, 32), seed=16, sm_scale=_INV(32), causal=True, window=16,
                          stride=8),
    "alibi_causal":  dict(shape=(1, 4, 96, 96, 32), seed=17, sm_scale=_INV(32), causal=True, alibi=True),
    "softcap":       dict(shape=(1, 2, 96, 96, 32), seed=18, sm_scale=1.0, softcap=5.0),
    "rect":          dict(shape=(1, 2, 64, 96, 32), seed=19, sm_scale=_INV(32)),
    "d64_causal":    dict(shape=(1, 1, 160, 160, 64), seed=20, sm_scale=_INV(64), causal=True),
}

# mask-factory fixtures: dense keep matrix and block-level predicate from the reference's masks.py
MASK_CASES = {
    "none":     dict(kind="none", seq=256, block_q=64, block_k=64),
    "causal":   dict(kind="causal", seq=256, block_q=64, block_k=32),
    "window":   dict(kind="sliding_window", seq=256, block_q=64, block_k=64, window=80),
    "document": dict(kind="document", seq=256, block_q=64, block_k=64, doc_lengths=[100, 28, 128]),
    "s2":       dict(kind="s2", seq=256, block_q=64, block_k=64, window=48, stride=32),
}


def make_inputs(c):
    """q, k, v, do as float32, drawn in that order from default_rng(seed)."""
    B, H, Sq, Sk, D = c["shape"]
    rng = np.random.default_rng(c["seed"])
    q = rng.standard_normal((B, H, Sq, D), dtype=np.float32)
    k = rng.standard_normal((B, H, Sk, D), dtype=np.float32)
    v = rng.standard_normal((B, H, Sk, D), dtype=np.float32)
    do = rng.standard_normal((B, H, Sq, D), dtype=np.float32)
    return q, k, v, do


def make_doc_ids(c):
    return np.stack([np.repeat(np.arange(len(ls), dtype=np.int32), ls) for ls in c["docs"]])


def slopes_for(c):
    H = c["shape"][1]
    return np.exp2(-8.0 * np.arange(1, H + 1) / H).astype(np.float32)


def alibi_bias(c):
    """ALiBi as a dense additive bias [B,H,Sq,Sk]: -slope_h * (i - j)."""
    B, H, Sq, Sk, _ = c["shape"]
    dist = (np.arange(Sq)[:, None] - np.arange(Sk)[None, :]).astype(np.float32)
    return np.broadcast_to(-slopes_for(c)[None, :, None, None] * dist, (B, H, Sq, Sk)).astype(np.float32).copy()
