"""The two tensor-core forward kernels against the CPU oracle, each FORCED through the environment switch the library
reads once per process (FLEXATTN_FWD_KERNEL=pair | pipe), so that both run on shapes where the other one would be
chosen: the two-query-tile kernel on short, ragged, rectangular and single-tile problems (odd tile counts leave its
second stream without a tile; a window or document mask gives the two streams different key ranges), the persistent
kernel on a long row."""
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
    from helpers import assert_close, make_qkvdo, oracle_hot_path, run_hot_path
    from oracle import mha_reference_cpu as oracle

    cases = %s
    for mask, score, Bn, H, Sq, Sk, D in cases:
        (q, k, v, do), host = make_qkvdo((Bn, H, Sq, D), (Bn, H, Sk, D), 11, torch.bfloat16)
        doc = oracle.draw_documents(np.random.default_rng(11), Bn, max(Sq, Sk), lo=60, hi=300)[0] if mask == "document" else None
        slopes = oracle.alibi_slopes(H) if score == "alibi" else None
        kw = dict(window=200 if "window" in mask else (96 if mask == "s2" else 0), stride=32 if mask == "s2" else 0)
        st = torch.zeros(4, dtype=torch.int32, device="cuda")
        sm = 1.0 / np.sqrt(D)
        got = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind=mask, score_kind=score, backend="tcgen05", doc_ids=doc,
                           cap=6.0, slopes=slopes, status=st, **kw)
        assert st.tolist() == [0, 0, 0, 0], (mask, score, st.tolist())
        want = oracle_hot_path(*host, sm_scale=sm, mask_kind=mask, score_kind=score, doc_ids=doc, cap=6.0, slopes=slopes,
                               window=kw["window"] or None, stride=kw["stride"] or None)
        assert_close(got, want, torch.bfloat16, what=f"forward kernel %s: {mask}/{score} {Sq}x{Sk} D{D}")
    # a seeded sweep of ragged shapes against the CUDA-core backend (same inputs, f32 arithmetic): the two streams of
    # the two-query-tile kernel meet every combination of key ranges here (one stream without tiles, ranges that
    # start or end a tile apart, documents that end inside a pair)
    rng = np.random.default_rng(2024)
    for it in range(%d):
        mask = ["none", "causal", "sliding_window", "sliding_window_causal", "document", "s2"][it %% 6]
        score = ["none", "alibi", "softcap"][int(rng.integers(3))]
        D = int(rng.choice([64, 128]))
        H = int(rng.integers(1, 4))
        Sq = int(rng.integers(1, 1300))
        # every query row keeps at least one key (rows without any are undefined, here and in the reference)
        Sk = int(rng.integers(1, 1300)) if mask == "none" else (Sq + int(rng.integers(0, 400)) if mask == "sliding_window" else Sq)
        (q, k, v, do), host = make_qkvdo((1, H, Sq, D), (1, H, Sk, D), 100 + it, torch.bfloat16)
        doc = oracle.draw_documents(np.random.default_rng(it), 1, max(Sq, Sk), lo=20, hi=400)[0] if mask == "document" else None
        slopes = oracle.alibi_slopes(H) if score == "alibi" else None
        kw = dict(window=int(rng.integers(1, 400)) if "window" in mask else (96 if mask == "s2" else 0), stride=32 if mask == "s2" else 0)
        st = torch.zeros(4, dtype=torch.int32, device="cuda")
        sm = 1.0 / np.sqrt(D)
        args = dict(sm_scale=sm, mask_kind=mask, score_kind=score, doc_ids=doc, cap=6.0, slopes=slopes, **kw)
        got = run_hot_path(fa, q, k, v, do, backend="tcgen05", status=st, **args)
        assert st.tolist() == [0, 0, 0, 0], (it, mask, score, Sq, Sk, st.tolist())
        want = run_hot_path(fa, q, k, v, do, backend="simt", **args)
        assert_close(got, want, torch.bfloat16, what=f"forward kernel %s sweep {it}: {mask}/{score} {Sq}x{Sk} D{D} H{H}", roundings=2)
    print("FWD_KERNEL_OK")
""")

PAIR_CASES = [("causal", "none", 2, 2, 777, 777, 128), ("document", "softcap", 2, 3, 500, 500, 64),
              ("none", "none", 1, 2, 300, 1000, 128), ("sliding_window_causal", "alibi", 1, 4, 900, 900, 128),
              ("s2", "none", 1, 2, 640, 640, 64), ("sliding_window", "none", 1, 2, 512, 768, 128),
              ("causal", "alibi", 1, 2, 1024, 1024, 64), ("causal", "softcap", 1, 2, 100, 100, 128),
              ("none", "alibi", 1, 2, 128, 1500, 128), ("document", "none", 1, 2, 1400, 1400, 128)]
PIPE_CASES = [("causal", "none", 1, 1, 4096, 4096, 128), ("none", "alibi", 1, 1, 200, 3300, 64)]


@pytest.mark.parametrize("kernel,cases,sweep", [("pair", PAIR_CASES, 36), ("pipe", PIPE_CASES, 12)])
def test_forced_forward_kernel_matches_the_oracle(kernel, cases, sweep):
    env = dict(os.environ, FLEXATTN_FWD_KERNEL=kernel)
    code = CHILD % (ROOT, os.path.join(ROOT, "tests"), repr(cases), kernel, sweep, kernel)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "FWD_KERNEL_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
