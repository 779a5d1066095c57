"""The CPU oracle against (1) fixtures produced by the reference's own mha_reference.py and
(2) an independent autograd check, since the reference pins no numbers itself."""
import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from golden_map import oracle_kwargs
from oracle import mha_reference_cpu as oracle


@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_matches_reference_vectors(name, golden):
    c = CASES[name]
    q, k, v, _ = make_inputs(c)
    o, l, m = oracle.mha_reference(q, k, v, save_residuals=True, block_rows=40, **oracle_kwargs(c))
    np.testing.assert_allclose(m, golden[f"{name}/m"], rtol=0, atol=2e-5)
    np.testing.assert_allclose(l, golden[f"{name}/l"], rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(o, golden[f"{name}/o"], rtol=0, atol=5e-6)


@pytest.mark.parametrize("name", sorted(n for n in CASES if not CASES[n].get("softcap")))
def test_backward_matches_reference_vectors(name, golden):
    c = CASES[name]
    q, k, v, do = make_inputs(c)
    dq, dk, dv = oracle.mha_bwd_reference(q, k, v, golden[f"{name}/o"], do, golden[f"{name}/l"],
                                          golden[f"{name}/m"], block_rows=40, **oracle_kwargs(c))
    np.testing.assert_allclose(dq, golden[f"{name}/dq"], rtol=0, atol=2e-5)
    np.testing.assert_allclose(dk, golden[f"{name}/dk"], rtol=0, atol=2e-5)
    np.testing.assert_allclose(dv, golden[f"{name}/dv"], rtol=0, atol=2e-5)


def _torch_attention(q, k, v, keep, sm_scale, score_kind, cap, slopes):
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * sm_scale
    if score_kind == "softcap":
        s = cap * torch.tanh(s / cap)
    if score_kind == "alibi":
        Sq, Sk = s.shape[-2:]
        dist = (torch.arange(Sq)[:, None] - torch.arange(Sk)[None, :]).double()
        s = s - torch.as_tensor(slopes).double()[None, :, None, None] * dist
    s = torch.where(keep, s, torch.full_like(s, -1e9))
    return torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, -1), v)


@pytest.mark.parametrize("score_kind", ["none", "softcap", "alibi"])
@pytest.mark.parametrize("mask_kind", ["causal", "document", "sliding_window_causal", "s2"])
def test_backward_matches_autograd_f64(mask_kind, score_kind):
    rng = np.random.default_rng(5)
    B, H, S, D = 2, 3, 70, 16
    q, k, v, do = (rng.standard_normal((B, H, S, D)).astype(np.float32) for _ in range(4))
    docs = np.stack([np.repeat(np.arange(3), [20, 30, 20]), np.repeat(np.arange(2), [45, 25])]).astype(np.int32)
    slopes = oracle.alibi_slopes(H)
    kw = dict(sm_scale=0.25, mask_kind=mask_kind, window=17, stride=8,
              doc_ids=docs if mask_kind == "document" else None,
              score_kind=score_kind, cap=3.0, alibi_slopes=slopes)
    o, l, m = oracle.mha_reference(q, k, v, save_residuals=True, block_rows=32, **kw)
    dq, dk, dv = oracle.mha_bwd_reference(q, k, v, o, do, l, m, block_rows=32, **kw)

    keep = np.stack([oracle.keep_mask(mask_kind, np.arange(S), np.arange(S), window=17, stride=8,
                                      doc_q=docs[b], doc_k=docs[b]) for b in range(B)])[:, None]
    tq, tk, tv = (torch.tensor(a, dtype=torch.float64, requires_grad=True) for a in (q, k, v))
    to = _torch_attention(tq, tk, tv, torch.tensor(keep), 0.25, score_kind, 3.0, slopes)
    to.backward(torch.tensor(do, dtype=torch.float64))
    np.testing.assert_allclose(o, to.detach().numpy(), atol=2e-5)
    np.testing.assert_allclose(dq, tq.grad.numpy(), atol=5e-5)
    np.testing.assert_allclose(dk, tk.grad.numpy(), atol=5e-5)
    np.testing.assert_allclose(dv, tv.grad.numpy(), atol=5e-5)


def test_delta_and_pairs():
    rng = np.random.default_rng(0)
    o, do = rng.standard_normal((2, 1, 2, 5, 8)).astype(np.float32)
    np.testing.assert_allclose(oracle.delta_reference(o, do), (o * do).sum(-1), rtol=1e-6)
    assert oracle.kept_pairs("causal", 512, 512) == [512 * 513 // 2]
    assert oracle.kept_pairs("sliding_window_causal", 8192, 8192, window=256) == [2064512]
    ids, lengths = oracle.draw_documents(np.random.default_rng(3), 2, 16384)
    assert ids.shape == (2, 16384) and all(sum(ls) == 16384 for ls in lengths)
    assert oracle.kept_pairs("document", 16384, 16384, doc_ids=ids) == \
        [sum(n * (n + 1) // 2 for n in ls) for ls in lengths]
