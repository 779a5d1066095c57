"""Turns the reference-style arguments (mask_fn / block_mask_fn / score_fn / causal / segment_ids) into a
bound ``Problem`` for the C ABI."""
from __future__ import annotations

import torch

from . import _binding as B
from . import masks, scores


def make_problem(q, k, *, ab, segment_ids, causal, sm_scale, mask_fn, block_mask_fn, score_fn, backend="auto",
                 status=None) -> B.Problem:
    if not isinstance(q, torch.Tensor):
        raise TypeError("flex attention expects torch CUDA tensors")
    mspec = masks.spec_of(mask_fn, block_mask_fn)
    sspec = scores.spec_of(score_fn)
    doc_ids = None
    if mspec is None:
        # the reference's kernels ignore `causal` and `segment_ids` (flex_attention_kernel.py:71-73); here
        # they select the causal / document mask when no mask callables are given
        if segment_ids is not None:
            mspec, doc_ids = masks.MaskSpec("document"), segment_ids
        elif causal:
            mspec = masks.MaskSpec("causal")
        else:
            mspec = masks.MaskSpec("none")
    elif mspec.kind == "document":
        if segment_ids is not None:
            doc_ids = segment_ids
        elif mspec.doc_lengths is not None:
            ids = masks.doc_ids_from_lengths(mspec.doc_lengths)
            need = max(q.shape[2], k.shape[2])
            if ids.shape[0] != need:
                raise ValueError(f"document lengths sum to {ids.shape[0]}, sequence length is {need}")
            doc_ids = torch.from_numpy(ids)
        else:
            raise ValueError("document mask needs doc_lengths or segment_ids")
    kw = dict(sm_scale=sm_scale, mask_kind=B.MASK_KIND_IDS[mspec.kind], window=mspec.window, stride=mspec.stride,
              doc_ids=doc_ids, backend=B.BACKEND_IDS[backend] if isinstance(backend, str) else backend,
              status=status, ab=ab)
    if sspec is not None:
        kw.update(score_kind=B.SCORE_KIND_IDS[sspec.kind], softcap=sspec.cap, alibi_slopes=sspec.slopes)
        if sspec.kind == "user":
            kw.update(user_score=B.user_score_handle(sspec.expr, sspec.dexpr))
    return B.Problem(q, k, **kw)
