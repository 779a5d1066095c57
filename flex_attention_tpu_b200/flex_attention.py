"""Differentiable flex attention: the forward, delta, dQ and dK/dV kernels tied together behind one call.

The reference wires only its plain flash attention into autodiff (``jax_exp.py:134-321``: ``flash_attention``
with ``jax.custom_vjp``, ``_flash_attention_fwd`` saving ``(q, k, v, ab, segment_ids, o, l, m)`` and
``_flash_attention_bwd`` calling the dkv and dq kernels); its flex kernels are only ever driven by hand
(``flex_attention_dq_bwd.py:905-945``).  This module is the same glue for the flex kernels, with
``torch.autograd.Function`` in the place of ``jax.custom_vjp``: residuals saved by the forward are exactly the
reference's, and the backward runs delta = rowsum(o * do), then dQ, then dK/dV.
"""
from __future__ import annotations

import torch

from ._resolve import make_problem


class _FlexAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ab, prob):
        o, l, m = prob.forward(q, k, v)
        ctx.save_for_backward(q, k, v, o, l, m)
        ctx.prob = prob
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, l, m = ctx.saved_tensors
        prob = ctx.prob
        do = do.contiguous()
        if prob.ab is not None and ctx.needs_input_grad[3]:
            _, dq, dk, dv, dab = prob.backward(q, k, v, o, do, l, m, want_dab=True)
            return dq, dk, dv, dab, None
        _, dq, dk, dv = prob.backward(q, k, v, o, do, l, m, need_dq=ctx.needs_input_grad[0],
                                      need_dkv=ctx.needs_input_grad[1] or ctx.needs_input_grad[2])
        return dq, dk, dv, None, None


def flex_attention_bwd(q, k, v, o, l, m, do, *, ab=None, segment_ids=None, causal: bool = False,
                       sm_scale: float = 1.0, mask_fns=None, score_fn=None, backend: str = "auto", two_streams=None):
    """The whole backward in one call: delta = rowsum(o * do), then dQ and dK/dV (launched on two streams so
    that the tail of one kernel overlaps the head of the other).  Residuals ``o, l, m`` as returned by
    ``_flex_attention_impl(..., save_residuals=True)``; the counterpart of the reference's
    ``_flash_attention_bwd`` (``jax_exp.py:276-321``).  ``two_streams=False`` keeps both kernels on the current
    stream.  Returns ``(dq, dk, dv)``."""
    mask_fn, block_mask_fn = mask_fns if mask_fns is not None else (None, None)
    prob = make_problem(q, k, ab=ab, segment_ids=segment_ids, causal=causal, sm_scale=sm_scale, mask_fn=mask_fn,
                        block_mask_fn=block_mask_fn, score_fn=score_fn, backend=backend)
    _, dq, dk, dv = prob.backward(q, k, v, o, do.contiguous(), l, m, two_streams=two_streams)
    return dq, dk, dv


def flex_attention(q, k, v, ab=None, segment_ids=None, *, causal: bool = False, sm_scale: float = 1.0,
                   mask_fns=None, score_fn=None, block_sizes=None, debug: bool = False, backend: str = "auto"):
    """softmax(mask(score_mod(sm_scale * q k^T))) v with gradients for q, k and v.

    Argument list after the reference's ``flash_attention`` (``jax_exp.py:143-155``), plus the two things that
    make it "flex": ``mask_fns`` = the ``(mask_fn, block_mask_fn)`` pair returned by a factory of ``masks`` and
    ``score_fn`` from ``scores``.  q, k, v: CUDA tensors ``[B, H, S, D]`` (bfloat16 or float32), contiguous.
    ``segment_ids``: ``[B, S]`` int32 document ids (selects the document mask when no ``mask_fns`` are given,
    as ``causal`` selects the causal one).  ``block_sizes`` / ``debug`` are accepted and ignored (tile sizes are
    fixed inside the kernels).  ``ab``: optional dense additive bias ``[B, H, Sq, Sk]`` (float32), added to
    the logits after the score function; it receives a gradient.  The same
    shape checks as the reference raise ``ValueError`` (``jax_exp.py:156-196``).
    """
    del block_sizes, debug
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be [batch, heads, seq, head_dim]")
    b, h, _, d = q.shape
    if k.shape[0] != b or v.shape[0] != b:
        raise ValueError(f"Batch size mismatch: got {b}, {k.shape[0]} and {v.shape[0]} (for q, k, v respectively)")
    if k.shape[1] != h or v.shape[1] != h:
        raise ValueError(f"Head count mismatch: got {h}, {k.shape[1]}, {v.shape[1]} (for q, k, v respectively)")
    if k.shape[3] != d:
        raise ValueError(f"Model dimension mismatch: got {d} and {k.shape[3]} (for q and k respectively)")
    if v.shape[3] != d:
        raise NotImplementedError("V model dimension unequal to KV model dimension unsupported")
    if k.shape[2] != v.shape[2]:
        raise ValueError(f"KV sequence length mismatch: got {k.shape[2]} and {v.shape[2]}")
    if ab is not None and tuple(ab.shape) != (b, h, q.shape[2], k.shape[2]):
        raise ValueError(f"Attention bias shape mismatch: expected {(b, h, q.shape[2], k.shape[2])}, got {tuple(ab.shape)}")
    mask_fn, block_mask_fn = mask_fns if mask_fns is not None else (None, None)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    prob = make_problem(q, k, ab=ab, segment_ids=segment_ids, causal=causal, sm_scale=sm_scale, mask_fn=mask_fn,
                        block_mask_fn=block_mask_fn, score_fn=score_fn, backend=backend)
    return _FlexAttentionFn.apply(q, k, v, ab, prob)
