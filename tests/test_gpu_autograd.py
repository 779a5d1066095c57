"""flex_attention: the autograd wrapper over fwd / delta / dQ / dK,dV (the glue the reference has for its plain
flash attention as jax.custom_vjp, jax_exp.py:134-321).  Gradients must be the kernels' own outputs, and match
the oracle."""
import numpy as np
import pytest
import torch

import workloads

from helpers import assert_close, make_qkvdo, oracle_hot_path, run_hot_path, build_mods


@pytest.mark.gpu
@pytest.mark.parametrize("mask_kind,score_kind,dtype", [("causal", "none", torch.bfloat16),
                                                         ("sliding_window_causal", "alibi", torch.bfloat16),
                                                         ("document", "softcap", torch.bfloat16),
                                                         ("causal", "softcap", torch.float32)])
def test_backward_through_autograd(mask_kind, score_kind, dtype):
    import flex_attention_tpu_b200 as fa
    B, H, S, D = 2, 3, 400, 64
    (q, k, v, do), host = make_qkvdo((B, H, S, D), (B, H, S, D), 21, dtype)
    doc = workloads.draw_documents(np.random.default_rng(3), B, S, lo=40, hi=200)[0] if mask_kind == "document" else None
    slopes = (2.0 ** (-8.0 * (np.arange(H) + 1) / H)).astype(np.float32) if score_kind == "alibi" else None
    kw = dict(sm_scale=0.11, mask_kind=mask_kind, score_kind=score_kind, window=96, doc_ids=doc, cap=6.0, slopes=slopes)
    mf, bf, sf, seg = build_mods(fa, mask_kind, score_kind, window=96, doc_ids=doc, cap=6.0, slopes=slopes)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = fa.flex_attention(qg, kg, vg, None, seg, sm_scale=0.11, mask_fns=None if mf is None else (mf, bf), score_fn=sf)
    o.backward(do)
    torch.cuda.synchronize()
    direct = run_hot_path(fa, q, k, v, do, **kw)
    for name, got in (("o", o), ("dq", qg.grad), ("dk", kg.grad), ("dv", vg.grad)):
        assert torch.equal(got.detach(), direct[name]), name
    okw = dict(kw)
    okw["window"], okw["cap"] = (96 if "window" in mask_kind else None), (6.0 if score_kind == "softcap" else None)
    want = oracle_hot_path(*host, **okw)
    got = dict(o=o.detach(), dq=qg.grad, dk=kg.grad, dv=vg.grad, l=direct["l"], m=direct["m"])
    assert_close(got, want, dtype, what=f"autograd {mask_kind}/{score_kind}")


@pytest.mark.gpu
def test_only_requested_gradients_are_computed():
    import flex_attention_tpu_b200 as fa
    (q, k, v, do), _ = make_qkvdo((1, 2, 256, 128), (1, 2, 256, 128), 5, torch.bfloat16)
    qg = q.clone().requires_grad_(True)
    fa.flex_attention(qg, k, v, causal=True, sm_scale=0.1).backward(do)
    assert qg.grad is not None and k.grad is None and v.grad is None


def test_shape_checks_raise_like_the_reference():
    """Argument validation happens before any device work (reference jax_exp.py:156-196)."""
    from flex_attention_tpu_b200.flex_attention import flex_attention
    q = torch.zeros(2, 4, 16, 64)
    with pytest.raises(ValueError, match="Batch size mismatch"):
        flex_attention(q, torch.zeros(3, 4, 16, 64), torch.zeros(2, 4, 16, 64))
    with pytest.raises(ValueError, match="Head count mismatch"):
        flex_attention(q, torch.zeros(2, 2, 16, 64), torch.zeros(2, 4, 16, 64))
    with pytest.raises(ValueError, match="Model dimension mismatch"):
        flex_attention(q, torch.zeros(2, 4, 16, 32), torch.zeros(2, 4, 16, 64))
    with pytest.raises(NotImplementedError):
        flex_attention(q, torch.zeros(2, 4, 16, 64), torch.zeros(2, 4, 16, 32))
    with pytest.raises(ValueError, match="KV sequence length mismatch"):
        flex_attention(q, torch.zeros(2, 4, 16, 64), torch.zeros(2, 4, 24, 64))
