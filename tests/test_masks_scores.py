"""Mask / score factories against fixtures produced by the reference's masks.py and against the oracle."""
import numpy as np
import pytest

from cases import MASK_CASES
from oracle import mha_reference_cpu as oracle


def _factory(fa, c):
    M = fa.masks
    bq, bk = c["block_q"], c["block_k"]
    return {"none": lambda: M.place_holder(bq, bk),
            "causal": lambda: M.make_causal_mask_fns(bq, bk),
            "sliding_window": lambda: M.make_sliding_window_mask_fns(bq, bk, c.get("window")),
            "document": lambda: M.make_jagged_mask_fns(bq, bk, c.get("doc_lengths")),
            "s2": lambda: M.make_s2_mask_fns(bq, bk, c.get("window"), c.get("stride"))}[c["kind"]]()


@pytest.mark.parametrize("name", sorted(MASK_CASES))
def test_mask_factories_match_reference_fixtures(name, golden):
    import flex_attention_tpu_b200 as fa
    c = MASK_CASES[name]
    mask_fn, block_fn = _factory(fa, c)
    s = c["seq"]
    idx = np.arange(s)
    want = np.unpackbits(golden[f"mask/{name}/dense"], axis=-1)[:, :s].astype(bool)
    if c["kind"] == "none":
        got = np.ones((s, s), bool)
    else:
        got = np.asarray(mask_fn(idx, idx), bool)
    assert (got == want).all()
    blocks = golden[f"mask/{name}/blocks"]
    for i in range(blocks.shape[0]):
        for j in range(blocks.shape[1]):
            assert bool(block_fn(i, j)) == bool(blocks[i, j]), (name, i, j)
    # the oracle's keep_mask agrees with the reference's element mask too
    docs = None
    if c["kind"] == "document":
        docs = fa.masks.doc_ids_from_lengths(c["doc_lengths"])
    keep = oracle.keep_mask(mask_fn.spec.kind, idx, idx, window=c.get("window"), stride=c.get("stride"), doc_q=docs,
                            doc_k=docs)
    assert (keep == want).all()
    assert mask_fn.spec == block_fn.spec and mask_fn.spec.kind == c["kind"]


def test_window_causal_extension_and_tags():
    import flex_attention_tpu_b200 as fa
    mf, bf = fa.masks.make_sliding_window_mask_fns(64, 64, 40, causal=True)
    idx = np.arange(200)
    want = oracle.keep_mask("sliding_window_causal", idx, idx, window=40)
    assert (np.asarray(mf(idx, idx)) == want).all()
    for i in range(4):
        for j in range(4):
            assert bool(bf(i, j)) == bool(want[i * 64:(i + 1) * 64, j * 64:(j + 1) * 64].any())
    assert mf.spec.kind == "sliding_window_causal" and mf.spec.window == 40


def test_score_factories():
    import flex_attention_tpu_b200 as fa
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((2, 16, 8)).astype(np.float32)
    sc = fa.scores.make_softcap_score_fn(5.0)
    np.testing.assert_allclose(sc(q, k), 5.0 * np.tanh(q @ k.T / 5.0), rtol=1e-6)
    al = fa.scores.make_alibi_score_fn([0.5, 0.25])
    dist = np.arange(16)[:, None] - np.arange(16)[None, :]
    np.testing.assert_allclose(al(q, k, head=1), q @ k.T - 0.25 * dist, rtol=1e-6)
    assert al.spec.kind == "alibi" and al.spec.slopes == (0.5, 0.25)
    np.testing.assert_allclose(fa.scores.alibi_slopes(8), oracle.alibi_slopes(8))
