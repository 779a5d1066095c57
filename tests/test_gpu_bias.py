"""Dense additive bias `ab` [B,H,Sq,Sk] (reference: flex_attention_kernel.py:262-266, mha_reference.py:50-51)
and its gradient `dab` ("dab is just ds", jax_exp.py:1676-1677), on the CUDA-core kernels (float32, and bfloat16
on request) and on the tensor-core kernels (bfloat16)."""
import numpy as np
import pytest
import torch

import workloads

from helpers import assert_close, build_mods, errors, make_qkvdo
from oracle import mha_reference_cpu as oracle

pytestmark = pytest.mark.gpu


def _run(fa, q, k, v, do, ab, *, sm_scale, mask_kind, score_kind, doc, cap, backend="auto", slopes=None):
    mf, bf, sf, seg = build_mods(fa, mask_kind, score_kind, doc_ids=doc, cap=cap, slopes=slopes)
    o, l, m = fa._flex_attention_impl(q, k, v, ab, seg, True, False, sm_scale, 1, 128, 128, 128, False, bf, mf, sf,
                                      backend=backend)
    delta = fa.bwd_preprocess(o, do)
    dq, dab = fa.flex_attention_bwd_dq(q, k, v, ab, seg, l, m, o, do, delta, sm_scale=sm_scale, score_fn=sf,
                                       mask_fn=mf, block_mask_fn=bf, return_dab=True, backend=backend)
    dk, dv = fa.flash_attention_bwd_dkv(k, v, q, ab, seg, l, m, delta, do, sm_scale=sm_scale, score_fn=sf,
                                        mask_fn=mf, block_mask_fn=bf, backend=backend)
    torch.cuda.synchronize()
    return dict(o=o, l=l, m=m, dq=dq, dk=dk, dv=dv, dab=dab)


@pytest.mark.parametrize("dtype,backend", [(torch.float32, "auto"), (torch.bfloat16, "simt"), (torch.bfloat16, "tcgen05")])
@pytest.mark.parametrize("mask_kind,score_kind", [("none", "none"), ("causal", "none"), ("document", "softcap")])
def test_bias_forward_and_backward(mask_kind, score_kind, dtype, backend):
    import flex_attention_tpu_b200 as fa
    B, H, Sq, Sk, D = 2, 3, 200, 333 if mask_kind == "none" else 200, 64
    (q, k, v, do), host = make_qkvdo((B, H, Sq, D), (B, H, Sk, D), 31, dtype)
    rng = np.random.default_rng(7)
    ab_h = (0.7 * rng.standard_normal((B, H, Sq, Sk))).astype(np.float32)
    ab = torch.from_numpy(ab_h).cuda()
    doc = workloads.draw_documents(np.random.default_rng(3), B, Sq, lo=30, hi=120)[0] if mask_kind == "document" else None
    cap = 5.0 if score_kind == "softcap" else 0.0
    got = _run(fa, q, k, v, do, ab, sm_scale=0.12, mask_kind=mask_kind, score_kind=score_kind, doc=doc, cap=cap,
               backend=backend)
    kw = dict(sm_scale=0.12, mask_kind=mask_kind, doc_ids=doc, score_kind=score_kind, cap=cap or None)
    qh, kh, vh, doh = host
    o, l, m = oracle.mha_reference(qh, kh, vh, ab_h, save_residuals=True, **kw)
    dq, dk, dv, dab = oracle.mha_bwd_reference(qh, kh, vh, o, doh, l, m, ab_h, return_dab=True, **kw)
    want = dict(o=o, l=l, m=m, dq=dq, dk=dk, dv=dv)
    assert_close(got, want, dtype, what=f"bias {mask_kind}/{score_kind}/{backend}")
    # dab is float32 in both cases; with bf16 inputs delta comes from the bf16-rounded o, hence the relative bound
    e = errors(got["dab"], dab)
    assert (e["max_abs"] <= 2e-3) if dtype == torch.float32 else (e["max_rel"] <= 1e-2), e


@pytest.mark.parametrize("mask_kind,score_kind,Sq,Sk,D", [("causal", "alibi", 777, 777, 128), ("none", "none", 300, 1000, 128),
                                                         ("sliding_window_causal", "softcap", 640, 640, 64),
                                                         ("document", "none", 1001, 1001, 128)])
def test_bias_on_the_tensor_core_kernels(mask_kind, score_kind, Sq, Sk, D):
    """Several kv tiles per row, ragged edges, odd row pitch of the bias (Sk not a multiple of 4: unaligned rows),
    masks that skip tiles (the bias gradient must be zero there) and every score functor."""
    import flex_attention_tpu_b200 as fa
    B, H = 2, 2
    (q, k, v, do), host = make_qkvdo((B, H, Sq, D), (B, H, Sk, D), 77, torch.bfloat16)
    rng = np.random.default_rng(11)
    ab_h = (0.7 * rng.standard_normal((B, H, Sq, Sk))).astype(np.float32)
    ab = torch.from_numpy(ab_h).cuda()
    doc = workloads.draw_documents(np.random.default_rng(3), B, Sq, lo=100, hi=400)[0] if mask_kind == "document" else None
    cap = 5.0 if score_kind == "softcap" else 0.0
    slopes = oracle.alibi_slopes(H) if score_kind == "alibi" else None
    window = 200 if mask_kind == "sliding_window_causal" else 0
    mf, bf, sf, seg = build_mods(fa, mask_kind, score_kind, window=window, doc_ids=doc, cap=cap, slopes=slopes)
    sm = 1.0 / np.sqrt(D)
    o, l, m = fa._flex_attention_impl(q, k, v, ab, seg, True, False, sm, 1, 128, 128, 128, False, bf, mf, sf, backend="tcgen05")
    delta = fa.bwd_preprocess(o, do)
    dq, dab = fa.flex_attention_bwd_dq(q, k, v, ab, seg, l, m, o, do, delta, sm_scale=sm, score_fn=sf, mask_fn=mf,
                                       block_mask_fn=bf, return_dab=True, backend="tcgen05")
    dk, dv = fa.flash_attention_bwd_dkv(k, v, q, ab, seg, l, m, delta, do, sm_scale=sm, score_fn=sf, mask_fn=mf,
                                        block_mask_fn=bf, backend="tcgen05")
    torch.cuda.synchronize()
    kw = dict(sm_scale=sm, mask_kind=mask_kind, doc_ids=doc, score_kind=score_kind, cap=cap or None, window=window or None,
              alibi_slopes=slopes)
    qh, kh, vh, doh = host
    ro, rl, rm = oracle.mha_reference(qh, kh, vh, ab_h, save_residuals=True, **kw)
    rdq, rdk, rdv, rdab = oracle.mha_bwd_reference(qh, kh, vh, ro, doh, rl, rm, ab_h, return_dab=True, **kw)
    assert_close(dict(o=o, l=l, m=m, dq=dq, dk=dk, dv=dv), dict(o=ro, l=rl, m=rm, dq=rdq, dk=rdk, dv=rdv), torch.bfloat16,
                 what=f"bias tcgen05 {mask_kind}/{score_kind}")
    assert bool(torch.isfinite(dab).all()), "every element of the dense bias gradient must be written"
    e = errors(dab, rdab)
    assert e["max_rel"] <= 1e-2, e


def test_bias_gets_a_gradient_through_autograd():
    import flex_attention_tpu_b200 as fa
    (q, k, v, do), _ = make_qkvdo((1, 2, 256, 128), (1, 2, 256, 128), 8, torch.bfloat16)
    ab = (0.5 * torch.randn(1, 2, 256, 256, device="cuda")).requires_grad_(True)
    qg = q.clone().requires_grad_(True)
    o = fa.flex_attention(qg, k, v, ab, causal=True, sm_scale=0.09)
    o.backward(do)
    assert ab.grad is not None and ab.grad.shape == ab.shape and qg.grad is not None
    # strictly upper-triangular pairs are masked: no gradient reaches the bias there
    assert float(ab.grad[0, 0].triu(1).abs().max()) == 0.0 and float(ab.grad.abs().max()) > 0.0
