"""User score functions on the GPU: a Python function traced by make_jax_score_fn, compiled into the tensor-core
forward, dQ and dK/dV kernels at run time, against the CPU oracle evaluating the SAME expression tree (and its
symbolic derivative) with NumPy."""
import numpy as np
import pytest
import torch

from helpers import assert_close, make_qkvdo, oracle_hot_path, run_hot_path
from oracle import mha_reference_cpu as oracle

pytestmark = pytest.mark.gpu


def _softcap(s, b, h, qi, ki):
    return 8.0 * np.tanh(s / 8.0)


def _distance_and_head(s, b, h, qi, ki):
    return s - 0.03 * (h + 1) * abs(qi - ki) + 0.25 * b


def _reference_form(q_tile, k_tile):
    from flex_attention_tpu_b200 import score_expr as se
    x = q_tile @ k_tile.T
    return se.where(x >= 0.0, x, 0.5 * x) + 0.1 * se.sigmoid(x)


# (the 1700-key unmasked and the 3300-key causal case are long enough for the two-query-tile forward kernel)
CASES = [("softcap", _softcap, "causal", 128, 777), ("distance", _distance_and_head, "none", 128, 500),
         ("distance", _distance_and_head, "document", 64, 700), ("leaky", _reference_form, "sliding_window_causal", 128, 640),
         ("distance", _distance_and_head, "none", 128, 1700), ("softcap", _softcap, "causal", 64, 3300)]


@pytest.mark.parametrize("name,fn,mask_kind,D,S", CASES)
def test_user_score_matches_the_oracle(name, fn, mask_kind, D, S):
    import flex_attention_tpu_b200 as fa
    B, H = (2, 3) if S < 1500 else (1, 2)
    (q, k, v, do), host = make_qkvdo((B, H, S, D), (B, H, S, D), 1200 + S, torch.bfloat16)
    sf = fa.util.make_jax_score_fn(fn)
    doc = oracle.draw_documents(np.random.default_rng(5), B, S, lo=60, hi=300)[0] if mask_kind == "document" else None
    window = 200 if mask_kind == "sliding_window_causal" else 0
    sm = 1.0 / np.sqrt(D)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    got = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind=mask_kind, score_kind="user", user_fn=sf, backend="tcgen05",
                       window=window, doc_ids=doc, status=status)
    assert status.tolist() == [0, 0, 0, 0], status.tolist()
    want = oracle_hot_path(*host, sm_scale=sm, mask_kind=mask_kind, score_kind="user", user=(sf, sf.dscore),
                           window=window or None, doc_ids=doc)
    assert_close(got, want, torch.bfloat16, what=f"user score {name}/{mask_kind}/D{D}")


def test_user_softcap_agrees_with_the_built_in_functor():
    import flex_attention_tpu_b200 as fa
    (q, k, v, do), _ = make_qkvdo((1, 4, 512, 128), (1, 4, 512, 128), 1300, torch.bfloat16)
    sm = 1.0 / np.sqrt(128)
    a = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", score_kind="user", backend="tcgen05",
                     user_fn=lambda s, b, h, qi, ki: 8.0 * np.tanh(s / 8.0))
    b_ = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", score_kind="softcap", cap=8.0, backend="tcgen05")
    for n in ("o", "dq", "dk", "dv"):     # tanhf against tanh.approx: a few bf16 ulps at most
        assert float((a[n].float() - b_[n].float()).abs().max()) <= 2e-2, n


def test_user_score_needs_the_tensor_core_kernels():
    import flex_attention_tpu_b200 as fa
    from flex_attention_tpu_b200._binding import FlexAttnError
    q = torch.randn(1, 1, 128, 64, device="cuda")
    sf = fa.util.make_jax_score_fn(_softcap)
    with pytest.raises(FlexAttnError):      # float32 inputs run on the CUDA-core kernels, which have no compiled user path
        fa._flex_attention_impl(q, q, q, None, None, True, True, 1.0, 1, 128, 128, 128, False, None, None, sf)
