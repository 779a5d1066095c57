"""The block-sparse mask map against a brute-force reduction of the oracle's keep matrix over each tile."""
import numpy as np
import pytest
import torch

from oracle import mha_reference_cpu as oracle

pytestmark = pytest.mark.gpu

CASES = [
    ("none", dict(), 300, 300),
    ("causal", dict(), 1000, 1000),
    ("causal", dict(), 384, 640),
    ("sliding_window", dict(window=200), 900, 900),
    ("sliding_window_causal", dict(window=256), 1536, 1536),
    ("sliding_window_causal", dict(window=100), 700, 700),
    ("s2", dict(window=130, stride=64), 1024, 1024),
    ("document", dict(), 1500, 1500),
]


@pytest.mark.parametrize("kind,kw,sq,sk", CASES)
def test_mask_map_matches_brute_force(kind, kw, sq, sk):
    from flex_attention_tpu_b200 import _binding as B
    batch = 2
    doc = None
    if kind == "document":
        rng = np.random.default_rng(7)
        doc, _ = oracle.draw_documents(rng, batch, max(sq, sk), lo=50, hi=400)
    q = torch.empty(batch, 1, sq, 64, dtype=torch.bfloat16, device="cuda")
    k = torch.empty(batch, 1, sk, 64, dtype=torch.bfloat16, device="cuda")
    prob = B.Problem(q, k, sm_scale=1.0, mask_kind=B.MASK_KIND_IDS[kind], window=kw.get("window", 0),
                     stride=kw.get("stride", 0), doc_ids=None if doc is None else torch.from_numpy(doc))
    T = B.TILE
    nq, nk = -(-sq // T), -(-sk // T)
    rows = batch if kind == "document" else 1
    for b in range(rows):
        keep = oracle.keep_mask(kind, np.arange(sq), np.arange(sk), window=kw.get("window"), stride=kw.get("stride"),
                                doc_q=None if doc is None else doc[b], doc_k=None if doc is None else doc[b])
        any_t = np.zeros((nq, nk), bool)
        all_t = np.zeros((nq, nk), bool)
        for i in range(nq):
            for j in range(nk):
                blk = keep[i * T:(i + 1) * T, j * T:(j + 1) * T]
                any_t[i, j] = blk.any()
                all_t[i, j] = blk.all() and (j + 1) * T <= sk      # ragged kv tiles always need the mask
        for which, n_self, any_m, all_m, other_len, n_other in (
                (0, nq, any_t, all_t, sk, nk),
                (1, nk, any_t.T, (np.array([[keep[i * T:(i + 1) * T, j * T:(j + 1) * T].all() and (i + 1) * T <= sq
                                             for i in range(nq)] for j in range(nk)])), sq, nq)):
            for t in range(n_self):
                lo, hi, flo, fhi = prob.read_map(which, b, t)
                listed = np.zeros(n_other, bool)
                listed[lo:hi] = True
                assert (listed | ~any_m[t]).all(), f"{kind} map {which} tile {t}: a tile with kept pairs is skipped"
                full = np.zeros(n_other, bool)
                full[flo:fhi] = True
                assert (~full | all_m[t]).all(), f"{kind} map {which} tile {t}: a partial tile is flagged full"
                assert lo <= flo <= fhi <= hi or flo == fhi
                if kind != "document":   # exactness: nothing listed that is empty, except inside the range
                    assert any_m[t][lo] if hi > lo else True
                    assert any_m[t][hi - 1] if hi > lo else True
