"""The bounds-checked build of the library (libflexattn_debug.so, selected with FLEXATTN_DEBUG=1): every direct
global-memory access of the tensor-core kernels is guarded and an index outside its array is reported through the
status words instead of faulting.  It stands in for a memory checker on this code: ragged and rectangular shapes,
every mask family, the dense bias and a run-time compiled score function run under it in a child process, must
leave the status words at zero and must still match the CPU oracle."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import sys
    sys.path.insert(0, %r); sys.path.insert(0, %r)
    import numpy as np, torch
    import flex_attention_tpu_b200 as fa
    from flex_attention_tpu_b200 import _binding as B
    from helpers import assert_close, make_qkvdo, oracle_hot_path, run_hot_path
    from oracle import mha_reference_cpu as oracle
    assert B.DEBUG_BUILD and B._LIB_PATH.endswith("libflexattn_debug.so")

    cases = [("causal", "none", 2, 2, 777, 777, 128), ("document", "softcap", 2, 3, 500, 500, 64),
             ("none", "none", 1, 2, 300, 1000, 128), ("sliding_window_causal", "alibi", 1, 4, 900, 900, 128),
             ("s2", "none", 1, 2, 640, 640, 64), ("causal", "user", 1, 2, 384, 384, 128)]
    for mask, score, Bn, H, Sq, Sk, D in cases:
        (q, k, v, do), host = make_qkvdo((Bn, H, Sq, D), (Bn, H, Sk, D), 5, torch.bfloat16)
        doc = oracle.draw_documents(np.random.default_rng(5), Bn, max(Sq, Sk), lo=60, hi=300)[0] if mask == "document" else None
        slopes = oracle.alibi_slopes(H) if score == "alibi" else None
        user = fa.util.make_jax_score_fn(lambda s, b, h, qi, ki: s - 0.02 * (h + 1) * abs(qi - ki)) if score == "user" else None
        kw = dict(window=200 if "window" in mask else (96 if mask == "s2" else 0), stride=32 if mask == "s2" else 0)
        st = torch.zeros(4, dtype=torch.int32, device="cuda")
        sm = 1.0 / np.sqrt(D)
        got = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind=mask, score_kind=score, backend="tcgen05", doc_ids=doc,
                           cap=6.0, slopes=slopes, status=st, user_fn=user, **kw)
        assert st.tolist() == [0, 0, 0, 0], (mask, score, st.tolist())
        want = oracle_hot_path(*host, sm_scale=sm, mask_kind=mask, score_kind=score, doc_ids=doc, cap=6.0, slopes=slopes,
                               window=kw["window"] or None, stride=kw["stride"] or None,
                               user=None if user is None else (user, user.dscore))
        assert_close(got, want, torch.bfloat16, what=f"debug build {mask}/{score}")
    # the dense bias and its gradient
    (q, k, v, do), host = make_qkvdo((1, 2, 300, 128), (1, 2, 333, 128), 6, torch.bfloat16)
    ab = (0.5 * torch.randn(1, 2, 300, 333, device="cuda"))
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    o, l, m = fa._flex_attention_impl(q, k, v, ab, None, True, False, 0.09, 1, 128, 128, 128, False, None, None, None,
                                      backend="tcgen05", status=st)
    d = fa.bwd_preprocess(o, do)
    dq, dab = fa.flex_attention_bwd_dq(q, k, v, ab, None, l, m, o, do, d, sm_scale=0.09, return_dab=True, backend="tcgen05", status=st)
    dk, dv = fa.flash_attention_bwd_dkv(k, v, q, ab, None, l, m, d, do, sm_scale=0.09, backend="tcgen05", status=st)
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0], st.tolist()
    assert all(bool(torch.isfinite(t.float()).all()) for t in (o, dq, dk, dv, dab))
    print("DEBUG_BUILD_OK")
""")


@pytest.mark.parametrize("fwd_kernel", ["", "pair"])
def test_bounds_checked_build_reports_nothing_and_matches_the_oracle(fwd_kernel):
    env = dict(os.environ, FLEXATTN_DEBUG="1")
    if fwd_kernel:  # the forward kernel for long rows, forced onto these short ones (where it can run)
        env["FLEXATTN_FWD_KERNEL"] = fwd_kernel
    r = subprocess.run([sys.executable, "-c", CHILD % (ROOT, os.path.join(ROOT, "tests"))], capture_output=True, text=True,
                       timeout=900, env=env)
    assert r.returncode == 0 and "DEBUG_BUILD_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
