"""Synthetic workload helpers for benchmarks and examples: document layouts, ALiBi slopes and the exact
number of kept (query, key) pairs of a mask, which is what the causal-adjusted FLOP counts are based on
(fwd 4*B*H*D*pairs, bwd 10*B*H*D*pairs; the reference counts 4*b*h*q*k*d and halves it for causal,
benchmark_fwd.py:20-21 and flex_attention_dq_bwd.py:618-626)."""
from __future__ import annotations

import numpy as np


def draw_documents(rng, batch, seq, lo=512, hi=4096):
    """Per batch row, document lengths uniform in [lo, hi] until they cover `seq` (last one truncated).
    Returns (doc_ids [batch, seq] int32, list of per-row length lists)."""
    ids = np.empty((batch, seq), np.int32)
    lengths_all = []
    for b in range(batch):
        lengths, total = [], 0
        while total < seq:
            n = min(int(rng.integers(lo, hi, endpoint=True)), seq - total)
            lengths.append(n)
            total += n
        ids[b] = np.repeat(np.arange(len(lengths), dtype=np.int32), lengths)
        lengths_all.append(lengths)
    return ids, lengths_all


def _run_lengths(row):
    row = np.asarray(row)
    edges = np.flatnonzero(np.diff(row)) + 1
    return np.diff(np.concatenate(([0], edges, [row.shape[0]])))


def kept_pairs(mask_kind, seq, *, window=0, stride=0, doc_ids=None):
    """Kept pairs per batch row for a square (seq x seq) problem: a list with one entry per row of
    `doc_ids` for the document mask (contiguous documents), else a single entry."""
    s = int(seq)
    if mask_kind == "none":
        return [s * s]
    if mask_kind == "causal":
        return [s * (s + 1) // 2]
    if mask_kind == "sliding_window_causal":
        w = min(int(window), s)
        return [w * (w + 1) // 2 + (s - w) * w]
    if mask_kind == "sliding_window":      # i - j < W, not causal
        w = int(window)
        return [sum(min(s, i + w) for i in range(s)) if w < s else s * s]
    if mask_kind == "document":
        d = np.asarray(doc_ids)
        d = d[None] if d.ndim == 1 else d
        return [int(sum(int(n) * (int(n) + 1) // 2 for n in _run_lengths(row))) for row in d]
    if mask_kind == "s2":
        w, st = int(window), int(stride)
        total = 0
        for i in range(s):
            local = min(i + 1, w)
            strided_old = 0 if i + 1 <= w else ((i - w) // st + 1)   # keys j <= i - w with j % st == 0
            total += local + strided_old
        return [total]
    raise ValueError(mask_kind)
