"""Forward + backward of the hot path for inputs that live in HOST memory.

The entry points of this package take device tensors, like the reference's take device arrays.  A caller
whose q, k, v, dO sit in (pinned) host memory pays for the PCIe transfers; done naively - copy everything
in, compute, copy everything out - the three phases run one after the other.  ``fwd_bwd_from_host`` splits
the batch (and, if asked, the heads of a batch row) into chunks and runs them through three CUDA streams
(host-to-device, compute, device-to-host) so that the copies of one chunk overlap the kernels of another and the
two copy directions overlap each other.  Every (batch, head) slice is independent, so chunking changes no result;
smaller chunks shorten the fill and the drain of the pipeline (the first copy in and the last copy out overlap
nothing).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import scores
from .flex_attention import flex_attention_bwd
from .flex_attention_kernel import _flex_attention_impl


_STREAMS = {}


def _streams(device):
    """Three long-lived side streams per device (copy in, compute, copy out).  They are reused across calls so
    that the caching allocator can recycle the per-stream buffers instead of allocating (and synchronising)
    on every call."""
    key = (device.type, device.index)
    if key not in _STREAMS:
        _STREAMS[key] = tuple(torch.cuda.Stream(device) for _ in range(3))
    return _STREAMS[key]


def fwd_bwd_from_host(q, k, v, do, *, sm_scale, mask_fn=None, block_mask_fn=None, score_fn=None, causal=False,
                      segment_ids=None, out: Optional[Sequence[torch.Tensor]] = None, chunk_batch: int = 1,
                      chunk_heads: Optional[int] = None, device: Optional[torch.device] = None, backend="auto"):
    """q, k, v, do: pinned host tensors [B, H, S, D].  Returns host tensors (o, dq, dk, dv) (``out`` if given:
    four pinned tensors that are overwritten).  ``segment_ids`` ([B, S], host or device) selects the document
    mask as in the entry points.  ``chunk_batch`` batch rows form a chunk; with ``chunk_batch == 1`` a chunk may be
    narrowed further to ``chunk_heads`` heads of one batch row (a contiguous block of host memory; ALiBi slopes
    are sliced with the heads; a user score function, which may depend on the head index, keeps whole rows).
    The call returns after everything has arrived in host memory."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H = q.shape[0], q.shape[1]
    sspec = scores.spec_of(score_fn)
    if chunk_heads is None or chunk_heads >= H or (sspec is not None and sspec.kind == "user"):
        chunk_heads = H
    if chunk_heads < H and chunk_batch != 1:
        raise ValueError("chunk_heads needs chunk_batch == 1 (a chunk must be one contiguous block of host memory)")
    if chunk_heads < 1:
        raise ValueError("chunk_heads must be positive")

    def score_for(h0, h1):
        """The score function of heads [h0, h1): per-head ALiBi slopes travel with their heads."""
        if sspec is None or sspec.kind != "alibi" or (h0 == 0 and h1 == H) or len(sspec.slopes) == 1:
            return score_fn
        return scores.make_alibi_score_fn(sspec.slopes[h0:h1])

    if out is None:
        out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, q, k, v)]
    o_h, dq_h, dk_h, dv_h = out
    seg_dev = None
    if segment_ids is not None:
        seg_dev = torch.as_tensor(segment_ids).to(device=device, dtype=torch.int32)
    cur = torch.cuda.current_stream(device)
    s_in, s_comp, s_out = _streams(device)
    for s in (s_in, s_comp, s_out):
        s.wait_stream(cur)
    slots = 2
    ev_comp_done = [None] * slots     # compute of the chunk that last used input slot i
    dev_in = [None] * slots
    keep = []
    chunks = [(b0, min(B, b0 + chunk_batch), h0, min(H, h0 + chunk_heads))
              for b0 in range(0, B, chunk_batch) for h0 in range(0, H, chunk_heads)]
    for ci, (b0, b1, h0, h1) in enumerate(chunks):
        slot = ci % slots
        sf = score_for(h0, h1)
        with torch.cuda.stream(s_in):
            if ev_comp_done[slot] is not None:
                s_in.wait_event(ev_comp_done[slot])          # the kernels that read this slot have finished
            if dev_in[slot] is None or dev_in[slot][0].shape[:2] != (b1 - b0, h1 - h0):
                dev_in[slot] = [torch.empty((b1 - b0, h1 - h0, *t.shape[2:]), dtype=t.dtype, device=device)
                                for t in (q, k, v, do)]
            for d, h_ in zip(dev_in[slot], (q, k, v, do)):
                d.copy_(h_[b0:b1, h0:h1], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in)
            qd, kd, vd, dod = dev_in[slot]
            seg = None if seg_dev is None else seg_dev[b0:b1].contiguous()
            o, l, m = _flex_attention_impl(qd, kd, vd, None, seg, True, causal, sm_scale, 1, 128, 128, 128, False,
                                           block_mask_fn, mask_fn, sf, backend=backend)
            dq, dk, dv = flex_attention_bwd(qd, kd, vd, o, l, m, dod, segment_ids=seg, causal=causal, sm_scale=sm_scale,
                                            mask_fns=None if mask_fn is None else (mask_fn, block_mask_fn),
                                            score_fn=sf, backend=backend, two_streams=False)
            delta = None
            ev_comp = torch.cuda.Event()
            ev_comp.record(s_comp)
            ev_comp_done[slot] = ev_comp
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp)
            for h_, r in zip((o_h, dq_h, dk_h, dv_h), (o, dq, dk, dv)):
                r.record_stream(s_out)
                h_[b0:b1, h0:h1].copy_(r, non_blocking=True)
        keep.append((o, l, m, delta, dq, dk, dv, seg))
    for s in (s_in, s_comp, s_out):
        cur.wait_stream(s)
    cur.synchronize()
    return o_h, dq_h, dk_h, dv_h
