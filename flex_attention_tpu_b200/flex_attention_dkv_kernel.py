"""dK/dV backward entry point with the reference's name and argument order
(reference ``flex_attention_dkv_kernel.py:23-174``; mask arguments as in its mask-aware twin
``flash_attention_dkv_bwd.py:27-47``)."""
from __future__ import annotations

from ._resolve import make_problem


def flash_attention_bwd_dkv(k, v, q, ab, segment_ids, l, m, di, do, *, block_b=None, block_q=None,
                            block_q_major=None, block_k_major=None, block_k=None, sm_scale=1.0, causal=False,
                            debug=False, score_fn=None, mask_fn=None, block_mask_fn=None, backend="auto",
                            status=None):
    """Returns ``(dk, dv)``: dv = p^T do and dk = sm_scale * (p * (do v^T - di) * score_mod'(s))^T q.

    Note the reference's argument order (k, v, q, ...).  ``di`` is delta = rowsum(o * do), [B, H, Sq]
    float32.  ``block_*`` / ``debug`` are ignored (fixed 128 x 128 tiles)."""
    del block_b, block_q, block_q_major, block_k_major, block_k, debug
    prob = make_problem(q, k, ab=ab, segment_ids=segment_ids, causal=causal, sm_scale=sm_scale, mask_fn=mask_fn,
                        block_mask_fn=block_mask_fn, score_fn=score_fn, backend=backend, status=status)
    return prob.bwd_dkv(q, k, v, do, l, m, di)
