"""dQ backward entry point with the reference's name and argument list
(reference ``flex_attention_dq_bwd.py:114-267``, ``flex_attention_bwd_dq``), plus the delta preprocess every
reference call site computes on the host before it (``flex_attention_dq_bwd.py:697``)."""
from __future__ import annotations

from ._resolve import make_problem


def bwd_preprocess(o, do):
    """delta = rowsum(o * do) as float32 [B, H, Sq], computed by the CUDA preprocess kernel."""
    prob = make_problem(o, o, ab=None, segment_ids=None, causal=False, sm_scale=1.0, mask_fn=None,
                        block_mask_fn=None, score_fn=None)
    return prob.preprocess(o, do)


def flex_attention_bwd_dq(q, k, v, ab, segment_ids, l, m, o, do, d, *, block_b=None, block_q=None,
                          block_k_major=None, block_k=None, sm_scale=1.0, debug=False, score_fn=None,
                          mask_fn=None, block_mask_fn=None, causal=False, backend="auto", status=None,
                          return_dab=False):
    """dq = sm_scale * (p * (do v^T - d) * score_mod'(s)) k, with p rebuilt from (l, m).

    ``ab``: optional dense additive bias [B, H, Sq, Sk] (float32).  With
    ``return_dab`` the call returns ``(dq, dab)``, dab = p * (do v^T - d), the gradient of ``ab``
    ("dab is just ds", reference ``jax_exp.py:1676-1677``).

    ``d`` is delta = rowsum(o * do) ([B, H, Sq] float32); pass ``None`` to have it computed here from
    ``o`` and ``do``.  ``o`` is otherwise unused, as in the reference kernel.  ``block_*`` / ``debug`` are
    ignored (fixed 128 x 128 tiles)."""
    del block_b, block_q, block_k_major, block_k, debug
    prob = make_problem(q, k, ab=ab, segment_ids=segment_ids, causal=causal, sm_scale=sm_scale, mask_fn=mask_fn,
                        block_mask_fn=block_mask_fn, score_fn=score_fn, backend=backend, status=status)
    if d is None:
        d = prob.preprocess(o, do)
    return prob.bwd_dq(q, k, v, do, l, m, d, want_dab=return_dab)
