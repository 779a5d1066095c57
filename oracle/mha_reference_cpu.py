"""CPU oracle for the flex-attention hot path (TEST INFRASTRUCTURE, not product code).

A NumPy float32 restatement of the reference's dense attention definitions:

* forward  : ``mha_reference``      follows reference ``mha_reference.py:5-109``
* backward : ``mha_bwd_reference``  follows reference ``mha_reference.py:112-237``
             (cross-checked with ``reference_bwd_test.py:640-707``: all-f32 math,
             ``ds * sm_scale``).
* delta    : ``delta_reference``    follows ``flex_attention_dq_bwd.py:697``.
* masks    : ``keep_mask``          follows ``masks.py:15-16`` (causal),
             ``masks.py:45-59`` (sliding window, *not* causal), ``masks.py:105-110``
             (document = same id and causal), ``masks.py:146-158`` (S2).

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module, and only as the
checker or the timed CPU baseline.  The product path never routes through it.

Parity pin: the reference holds no golden vectors and JAX (its only runtime) is not
installed, so the reference's Pallas kernels are *unpinned*.  The dense definitions
above are pinned indirectly: ``tests/golden/make_golden.py`` executes the reference's
own ``mha_reference.py`` source with NumPy standing in for ``jax.numpy`` and commits
the outputs; ``tests/test_oracle.py`` checks this file against those fixtures.

Conventions fixed by this build (the reference is self-inconsistent about where
``sm_scale`` is applied when a score function is present; the choices coincide with the
reference whenever ``sm_scale == 1``):

    s      = sm_scale * <q_i, k_j>
    t      = score_mod(s) + bias            softcap: cap*tanh(s/cap); ALiBi: bias=-slope_h*(i-j)
    x      = t if keep(i, j) else -1e9      (``mha_reference.py:62,77,94`` *replace* with -1e9)
    m_i    = max_j x ; l_i = sum_j exp(x - m_i) ; p = exp(x - m_i) / l_i
    o_i    = sum_j p_ij v_j
    dt     = p * (do.v^T - delta) ; ds = dt * score_mod'(s)
    dq     = sm_scale * ds @ k ; dk = sm_scale * ds^T @ q ; dv = p^T @ do

The work is row-blocked over queries so that S = 32768 needs O(block * S) memory.
"""
from __future__ import annotations

import numpy as np

MASK_VALUE = np.float32(-1e9)  # mha_reference.py:62

MASK_KINDS = ("none", "causal", "sliding_window", "sliding_window_causal", "document", "s2")
SCORE_KINDS = ("none", "alibi", "softcap", "user")


def keep_mask(kind, q_idx, k_idx, *, window=None, stride=None, doc_q=None, doc_k=None):
    """Boolean [len(q_idx), len(k_idx)] matrix, True = keep.  See module docstring for sources."""
    qi = np.asarray(q_idx, dtype=np.int64)[:, None]
    kj = np.asarray(k_idx, dtype=np.int64)[None, :]
    if kind == "none":
        return np.ones((qi.shape[0], kj.shape[1]), dtype=bool)
    if kind == "causal":
        return qi >= kj
    if kind == "sliding_window":          # masks.py:45-59: only the "too old" bound
        return (qi - kj) < window
    if kind == "sliding_window_causal":   # mha_reference.py:59-62 + 80-94
        d = qi - kj
        return (d >= 0) & (d < window)
    if kind == "document":                # masks.py:105-110
        return (np.asarray(doc_q)[:, None] == np.asarray(doc_k)[None, :]) & (qi >= kj)
    if kind == "s2":                      # masks.py:146-158
        d = qi - kj
        return ((d >= 0) & (d < window)) | ((kj % stride == 0) & (qi >= kj))
    raise ValueError(f"unknown mask kind {kind!r}")


def _kv_limit(kind, q_hi, sk):
    """Exclusive upper bound on key positions any row < q_hi can keep (skips all-masked columns;
    a masked column contributes exp(-1e9 - m) == 0 exactly in f32, so the result is unchanged)."""
    if kind in ("causal", "sliding_window_causal", "document", "s2"):
        return min(sk, q_hi)
    return sk


def _logits_block(qb, k, *, sm_scale, score_kind, cap, slope, q0, mask_kind, window, stride,
                  doc_q, doc_k, ab_block, user=None, b=0, h=0):
    """Rows [q0, q0+len(qb)) of the masked logits plus what the backward needs to redo score_mod."""
    s = (qb @ k.T) * np.float32(sm_scale)
    dsig = None
    if score_kind == "softcap":
        th = np.tanh(s / np.float32(cap))
        t = np.float32(cap) * th
        dsig = np.float32(1.0) - th * th
    else:
        t = s
    nq, nk = s.shape
    q_idx = np.arange(q0, q0 + nq)
    k_idx = np.arange(nk)
    if score_kind == "user":
        # any score function of the scaled score, batch, head and positions (the reference's score_fn branch,
        # mha_reference.py:44-48, generalised); its derivative plays the part jax.vjp plays in the reference
        f, df = user
        t = np.asarray(f(s, b, h, q_idx[:, None], k_idx[None, :]), np.float32)
        dsig = np.asarray(df(s, b, h, q_idx[:, None], k_idx[None, :]), np.float32) * np.ones_like(s)
    if score_kind == "alibi":
        dist = (q_idx[:, None] - k_idx[None, :]).astype(np.float32)
        t = t - np.float32(slope) * dist
    if ab_block is not None:
        t = t + ab_block
    keep = keep_mask(mask_kind, q_idx, k_idx, window=window, stride=stride,
                     doc_q=None if doc_q is None else doc_q[q0:q0 + nq],
                     doc_k=None if doc_k is None else doc_k[:nk])
    x = np.where(keep, t, MASK_VALUE).astype(np.float32)
    return x, dsig


def _per_head_args(b, h, score_kind, alibi_slopes, doc_ids, ab):
    slope = None
    if score_kind == "alibi":
        slope = float(np.asarray(alibi_slopes, dtype=np.float32)[h])
    docs = None
    if doc_ids is not None:
        d = np.asarray(doc_ids)
        docs = d if d.ndim == 1 else d[b]
    abh = None if ab is None else ab[b, h]
    return slope, docs, abh


def mha_reference(q, k, v, ab=None, *, sm_scale=1.0, save_residuals=False,
                  mask_kind="none", window=None, stride=None, doc_ids=None,
                  score_kind="none", cap=None, alibi_slopes=None, block_rows=1024, user=None):
    """Dense forward.  q,k,v: [B,H,S,D] arrays (any float dtype; computed in f32).

    Returns ``o`` (f32) or ``(o, l, m)`` with l = sum exp(x - m), m = row max, both [B,H,Sq] f32
    (the reference's residual pair, ``mha_reference.py:99-109``)."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    o = np.empty((B, H, Sq, D), np.float32)
    l = np.empty((B, H, Sq), np.float32)
    m = np.empty((B, H, Sq), np.float32)
    for b in range(B):
        for h in range(H):
            slope, docs, abh = _per_head_args(b, h, score_kind, alibi_slopes, doc_ids, ab)
            for q0 in range(0, Sq, block_rows):
                q1 = min(Sq, q0 + block_rows)
                kl = _kv_limit(mask_kind, q1, Sk)
                x, _ = _logits_block(q[b, h, q0:q1], k[b, h, :kl], sm_scale=sm_scale,
                                     score_kind=score_kind, cap=cap, slope=slope, q0=q0,
                                     mask_kind=mask_kind, window=window, stride=stride,
                                     doc_q=docs, doc_k=docs,
                                     ab_block=None if abh is None else abh[q0:q1, :kl], user=user, b=b, h=h)
                mb = x.max(axis=-1)
                un = np.exp(x - mb[:, None])
                lb = un.sum(axis=-1, dtype=np.float32)
                l_safe = np.where(lb == 0, np.float32(1.0), lb)      # mha_reference.py:104
                o[b, h, q0:q1] = (un / l_safe[:, None]) @ v[b, h, :kl]
                l[b, h, q0:q1] = lb
                m[b, h, q0:q1] = mb
    return (o, l, m) if save_residuals else o


def delta_reference(o, do):
    """delta = rowsum(o * do) in f32 (``flex_attention_dq_bwd.py:697``)."""
    return (np.asarray(o, np.float32) * np.asarray(do, np.float32)).sum(axis=-1, dtype=np.float32)


def mha_bwd_reference(q, k, v, o, do, l, m, ab=None, *, sm_scale=1.0,
                      mask_kind="none", window=None, stride=None, doc_ids=None,
                      score_kind="none", cap=None, alibi_slopes=None, block_rows=1024, return_dab=False, user=None):
    """Dense backward mirroring ``mha_reference.py:112-237``.  Returns (dq, dk, dv) in f32, plus the gradient of
    the dense bias ``ab`` ([B,H,Sq,Sk]) with ``return_dab``."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    o = np.asarray(o, dtype=np.float32)
    do = np.asarray(do, dtype=np.float32)
    l = np.asarray(l, dtype=np.float32)
    m = np.asarray(m, dtype=np.float32)
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    dq = np.zeros((B, H, Sq, D), np.float32)
    dk = np.zeros((B, H, Sk, D), np.float32)
    dv = np.zeros((B, H, Sk, D), np.float32)
    dab = np.zeros((B, H, Sq, Sk), np.float32) if return_dab else None
    c = np.float32(sm_scale)
    for b in range(B):
        for h in range(H):
            slope, docs, abh = _per_head_args(b, h, score_kind, alibi_slopes, doc_ids, ab)
            for q0 in range(0, Sq, block_rows):
                q1 = min(Sq, q0 + block_rows)
                kl = _kv_limit(mask_kind, q1, Sk)
                x, dsig = _logits_block(q[b, h, q0:q1], k[b, h, :kl], sm_scale=sm_scale,
                                        score_kind=score_kind, cap=cap, slope=slope, q0=q0,
                                        mask_kind=mask_kind, window=window, stride=stride,
                                        doc_q=docs, doc_k=docs,
                                        ab_block=None if abh is None else abh[q0:q1, :kl], user=user, b=b, h=h)
                lb = l[b, h, q0:q1]
                l_safe = np.where(lb == 0, np.float32(1.0), lb)       # mha_reference.py:206
                p = np.exp(x - m[b, h, q0:q1, None]) / l_safe[:, None]
                dob = do[b, h, q0:q1]
                dv[b, h, :kl] += p.T @ dob                             # :213
                dp = dob @ v[b, h, :kl].T                              # :216
                sum_d = (dob * o[b, h, q0:q1]).sum(axis=-1, dtype=np.float32)  # :220
                ds = p * (dp - sum_d[:, None])                         # :221
                if dab is not None:
                    dab[b, h, q0:q1, :kl] = ds                         # "dab is just ds", jax_exp.py:1676-1677
                if dsig is not None:
                    ds = ds * dsig
                ds = ds * c                                            # :229
                dq[b, h, q0:q1] = ds @ k[b, h, :kl]                    # :230
                dk[b, h, :kl] += ds.T @ q[b, h, q0:q1]                 # :231
    return (dq, dk, dv, dab) if return_dab else (dq, dk, dv)


# ----------------------------------------------------------------------------------------------
# Workload helpers shared by the tests and the bench (synthetic inputs, exact work counts).
# ----------------------------------------------------------------------------------------------

def alibi_slopes(num_heads):
    """slope_h = 2^(-8 (h+1) / H), the standard ALiBi schedule."""
    h = np.arange(1, num_heads + 1, dtype=np.float64)
    return np.exp2(-8.0 * h / num_heads).astype(np.float32)


def draw_documents(rng, batch, seq, lo=512, hi=4096):
    """Per batch row, document lengths uniform in [lo, hi] until they cover ``seq`` (last truncated).
    Returns (doc_ids [B,S] int32, list of length lists)."""
    ids = np.empty((batch, seq), np.int32)
    all_lengths = []
    for b in range(batch):
        lengths, total = [], 0
        while total < seq:
            n = int(rng.integers(lo, hi, endpoint=True))
            n = min(n, seq - total)
            lengths.append(n)
            total += n
        ids[b] = np.repeat(np.arange(len(lengths), dtype=np.int32), lengths)
        all_lengths.append(lengths)
    return ids, all_lengths


def kept_pairs(mask_kind, sq, sk, *, window=None, stride=None, doc_ids=None):
    """Exact number of kept (q, k) pairs per batch row: list of ints (length B, or 1 without docs)."""
    if mask_kind == "document":
        d = np.asarray(doc_ids)
        d = d[None] if d.ndim == 1 else d
        out = []
        for row in d:
            total = 0
            # generic (ids need not be sorted): count pairs i>=j with equal id, blockwise
            for q0 in range(0, sq, 2048):
                q1 = min(sq, q0 + 2048)
                kl = min(sk, q1)
                total += int(keep_mask("document", np.arange(q0, q1), np.arange(kl),
                                       doc_q=row[q0:q1], doc_k=row[:kl]).sum())
            out.append(total)
        return out
    total = 0
    for q0 in range(0, sq, 2048):
        q1 = min(sq, q0 + 2048)
        total += int(keep_mask(mask_kind, np.arange(q0, q1), np.arange(sk), window=window,
                               stride=stride).sum())
    return [total]
