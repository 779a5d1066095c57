"""User score functions, the part that needs no GPU: tracing a Python function into an expression tree, its
symbolic derivative, the CUDA text, and the run-time compilation of the three tensor-core kernels around it
(NVRTC produces the sm_100a cubin without a device; loading and launching are covered by the GPU tests)."""
import ctypes

import numpy as np
import pytest

from flex_attention_tpu_b200 import score_expr as se


def _env(n=7):
    return dict(s=np.linspace(-3, 3, n).astype(np.float32), b=1, h=2, q_idx=np.arange(n) + 5, k_idx=np.arange(n)[::-1].copy())


FUNCS = {
    "softcap": lambda s, b, h, qi, ki: 20.0 * se.tanh(s / 20.0),
    "numpy_namesakes": lambda s, b, h, qi, ki: np.tanh(s) * 3.0 + np.maximum(s, 0.0) - np.abs(s) * 0.5,
    "positions": lambda s, b, h, qi, ki: s - 0.05 * (h + 1) * abs(qi - ki) + 0.01 * b,
    "where_and_powers": lambda s, b, h, qi, ki: se.where(s >= 0.0, s ** 2, -0.1 * s) + se.sigmoid(s) * se.sqrt(s * s + 1.0),
    "reference_form": lambda q, k: 30.0 * se.tanh((q @ k.T) / 30.0),
    "string": "s * exp(-0.001 * abs(q_idx - k_idx)) + log(1.0 + s * s)",
}


@pytest.mark.parametrize("name", sorted(FUNCS))
def test_trace_evaluate_and_differentiate(name):
    e, d = se.trace(FUNCS[name])
    env = _env()
    val = se.evaluate(e, env)
    assert np.isfinite(val).all() and val.shape == env["s"].shape
    if name == "softcap":
        np.testing.assert_allclose(val, 20.0 * np.tanh(env["s"] / 20.0), rtol=1e-6)
    # derivative against central differences of the traced value, away from the kinks at s == 0
    eps = 1e-2
    hi = se.evaluate(e, dict(env, s=env["s"] + eps)).astype(np.float64)
    lo = se.evaluate(e, dict(env, s=env["s"] - eps)).astype(np.float64)
    smooth = np.abs(env["s"]) > 2 * eps
    np.testing.assert_allclose(se.evaluate(d, env)[smooth], ((hi - lo) / (2 * eps))[smooth], rtol=2e-2, atol=2e-3)
    text = se.to_cuda(e)
    assert text.count("(") == text.count(")") and "q_idx" not in text


def test_what_cannot_be_traced_is_refused():
    import flex_attention_tpu_b200 as fa
    with pytest.raises(TypeError):
        se.trace(lambda q, k: q + 1)                    # tiles only support q @ k.T
    with pytest.raises(TypeError):
        se.trace(lambda s, b, h, qi, ki: s if s > 0 else -s)   # data-dependent Python control flow
    with pytest.raises(TypeError):
        se.trace(lambda s: s)                           # neither of the two signatures
    with pytest.raises(NotImplementedError):
        fa.util.make_jax_score_fn(lambda a, b: a @ b.T @ a)
    sf = fa.util.make_jax_score_fn(FUNCS["positions"])
    assert sf.spec.kind == "user" and "fabsf" in sf.spec.expr
    np.testing.assert_allclose(sf(np.float32(1.5), 0, 1, 10, 4), 1.5 - 0.05 * 2 * 6, rtol=1e-6)
    assert fa.util.make_jax_score_fn(sf) is sf          # already traced: passes through


def test_kernels_compile_around_a_user_function_without_a_gpu():
    from flex_attention_tpu_b200 import _binding as B
    import flex_attention_tpu_b200 as fa
    sf = fa.scores.make_user_score_fn(FUNCS["positions"])
    h = B.user_score_handle(sf.spec.expr, sf.spec.dexpr)
    assert h > 0 and B.user_score_handle(sf.spec.expr, sf.spec.dexpr) == h
    rc = B.lib.flexattn_user_score_compile(h, 0, 128, B.MASK_CAUSAL)
    if rc == 12:
        pytest.skip("libnvrtc is not installed here")
    assert rc == 0, B.lib.flexattn_user_score_log(h).decode()
    assert B.lib.flexattn_user_score_compile(h, 1, 64, B.MASK_DOCUMENT) == 0
    assert B.lib.flexattn_user_score_compile(h, 2, 128, B.MASK_SLIDING_WINDOW_CAUSAL) == 0
    assert B.lib.flexattn_user_score_compile(h, 3, 128, B.MASK_CAUSAL) == 0   # the forward kernel for long rows
    assert B.lib.flexattn_user_score_compile(h, 4, 128, 0) == 7 and B.lib.flexattn_user_score_compile(h, 0, 96, 0) == 4
    # an expression that is not CUDA: refused with the compiler's message, the library stays usable
    bad = ctypes.c_int32(0)
    assert B.lib.flexattn_user_score_create(b"s +* undefined_thing", b"1.0f", ctypes.byref(bad)) == 0
    assert B.lib.flexattn_user_score_compile(bad.value, 0, 128, 0) == 13
    assert b"error" in B.lib.flexattn_user_score_log(bad.value)
    assert B.lib.flexattn_user_score_destroy(bad.value) == 0 and B.lib.flexattn_user_score_destroy(bad.value) == 7
    # the plain entry points validate the handle before anything else happens
    p = B.FlexAttnParams()
    p.batch, p.heads, p.seq_q, p.seq_k, p.head_dim, p.score_kind = 1, 1, 128, 128, 128, B.SCORE_USER
    assert B.lib.flexattn_fwd(None, ctypes.byref(p)) == 7          # no handle
