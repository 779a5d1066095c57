"""Forward entry point with the reference's name and argument list
(reference ``flex_attention_kernel.py:66-193``, ``_flex_attention_impl``)."""
from __future__ import annotations

from ._resolve import make_problem


def _flex_attention_impl(q, k, v, ab, segment_ids, save_residuals, causal, sm_scale, block_b, block_q,
                         block_k_major, block_k, debug, block_mask_fn, mask_fn, score_fn, *, backend="auto",
                         status=None):
    """softmax(mask(score_mod(sm_scale * q k^T))) v on the GPU.

    q, k, v: torch CUDA tensors [B, H, S, D], bfloat16 or float32.  Returns ``o`` or, with
    ``save_residuals``, ``(o, l, m)`` with l = sum exp(x - m) and m = row max, both [B, H, Sq] float32,
    as the reference does (flex_attention_kernel.py:189-193).

    ``block_*`` and ``debug`` are accepted for signature compatibility and ignored: tile sizes are fixed
    inside the kernels (128 x 128).  ``mask_fn`` / ``block_mask_fn`` / ``score_fn`` must come from
    ``masks`` / ``scores`` of this package.  Differences from the reference, all no-ops for the calls it
    makes itself: ``sm_scale`` is applied before the score function (the reference skips it when a
    score_fn is present and only tests sm_scale == 1), and ``causal`` / ``segment_ids`` select a mask when
    no mask callables are passed instead of being ignored.
    """
    del block_b, block_q, block_k_major, block_k, debug
    prob = make_problem(q, k, ab=ab, segment_ids=segment_ids, causal=causal, sm_scale=sm_scale, mask_fn=mask_fn,
                        block_mask_fn=block_mask_fn, score_fn=score_fn, backend=backend, status=status)
    o, l, m = prob.forward(q, k, v)
    return (o, l, m) if save_residuals else o
