"""fwd_bwd_from_host: pinned host buffers in and out, chunks of the batch pipelined through copy and compute
streams.  Must give exactly what the device-tensor entry points give on the whole batch."""
import numpy as np
import pytest
import torch

from helpers import make_qkvdo, run_hot_path

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mask_kind,score_kind", [("causal", "none"), ("document", "softcap"), ("causal", "alibi")])
def test_host_pipeline_matches_device_entry_points(mask_kind, score_kind):
    import flex_attention_tpu_b200 as fa
    from flex_attention_tpu_b200 import host_api
    import workloads
    B, H, S, D = 5, 4, 640, 128
    (q, k, v, do), _ = make_qkvdo((B, H, S, D), (B, H, S, D), 77, torch.bfloat16)
    doc = None
    if mask_kind == "document":
        doc, _ = workloads.draw_documents(np.random.default_rng(1), B, S, lo=60, hi=300)
    slopes = fa.scores.alibi_slopes(H) if score_kind == "alibi" else None
    want = run_hot_path(fa, q, k, v, do, sm_scale=0.09, mask_kind=mask_kind, score_kind=score_kind, doc_ids=doc, cap=7.0,
                        slopes=slopes)
    host = [t.cpu().pin_memory() for t in (q, k, v, do)]
    mf = bf = sf = None
    if mask_kind == "causal":
        mf, bf = fa.masks.make_causal_mask_fns(128, 128)
    if score_kind == "softcap":
        sf = fa.scores.make_softcap_score_fn(7.0)
    if score_kind == "alibi":
        sf = fa.scores.make_alibi_score_fn(slopes)
    for chunk, heads in ((1, None), (2, None), (5, None), (1, 1), (1, 3)):     # the last: chunks of 3 heads and of 1
        o, dq, dk, dv = host_api.fwd_bwd_from_host(*host, sm_scale=0.09, mask_fn=mf, block_mask_fn=bf, score_fn=sf,
                                                   segment_ids=None if doc is None else torch.from_numpy(doc),
                                                   chunk_batch=chunk, chunk_heads=heads)
        for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
            assert not got.is_cuda and got.is_pinned()
            assert torch.equal(got, want[name].cpu()), (name, chunk, heads)
