"""Generate the golden fixtures in this folder from the reference's own Python sources.

Run once in a container that has the reference checkout (it does not travel to the GPU box):

    python tests/golden/make_golden.py /path/to/reference

JAX is not installed in the build image, so the reference's dense definitions
(``mha_reference.py``), mask factories (``masks.py``) and score factories (``scores.py``) are
imported with NumPy standing in for ``jax.numpy`` (they only use ``einsum / where / exp / max /
sum / arange / abs / tanh / dot / maximum / minimum``, which NumPy provides with the same
semantics) and a two-line ``jax.vmap`` stand-in that loops over the leading axis.  ``util`` (the
AST rewriter, which needs JAX internals and is unused by ``mha_reference``) is replaced by an
empty stub.  The arithmetic that produces the fixtures is therefore the reference's own source,
executed in IEEE float32 by NumPy.

Inputs are NOT stored: every case regenerates them from its seed with
``numpy.random.default_rng(seed).standard_normal`` in the order q, k, v, do (see ``cases.py``).
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, MASK_CASES, make_inputs, make_doc_ids, alibi_bias  # noqa: E402


def _install_shims():
    jax = types.ModuleType("jax")
    jax.Array = np.ndarray
    jax.numpy = np

    def vmap(fn, in_axes=(0, 0)):
        def batched(a, b):
            return np.stack([fn(x, y) for x, y in zip(a, b)])
        return batched

    jax.vmap = vmap
    util = types.ModuleType("util")
    util.make_jax_score_fn = lambda f: f
    sys.modules["jax"] = jax
    sys.modules["jax.numpy"] = np
    sys.modules["util"] = util


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    ref_dir = sys.argv[1]
    _install_shims()
    sys.path.insert(0, ref_dir)
    import mha_reference as ref      # noqa: E402  (reference mha_reference.py)
    import masks as ref_masks        # noqa: E402  (reference masks.py)
    import scores as ref_scores      # noqa: E402  (reference scores.py)

    out = {}
    for name, c in CASES.items():
        q, k, v, do = make_inputs(c)
        kw = dict(sm_scale=c["sm_scale"], causal=c.get("causal", False),
                  window_size=c.get("window"), s2_stride=c.get("stride"))
        if c.get("docs"):
            kw["segment_ids"] = make_doc_ids(c)
        ab = alibi_bias(c) if c.get("alibi") else None
        if c.get("softcap"):
            kw["score_fn"] = ref_scores.make_softcap_score_fn(c["softcap"])
        o, l, m = ref.mha_reference(q, k, v, None if ab is None else ab.copy(),
                                    save_residuals=True, **kw)
        out[f"{name}/o"], out[f"{name}/l"], out[f"{name}/m"] = o, l, m
        if not c.get("softcap"):        # the reference's score_fn backward needs jax.vjp
            dq, dk, dv = ref.mha_bwd_reference(q, k, v, o, do, l, m, ab, **kw)
            out[f"{name}/dq"], out[f"{name}/dk"], out[f"{name}/dv"] = dq, dk, dv

    for name, c in MASK_CASES.items():
        bq, bk, s = c["block_q"], c["block_k"], c["seq"]
        if c["kind"] == "causal":
            mask_fn, block_fn = ref_masks.make_causal_mask_fns(bq, bk)
        elif c["kind"] == "sliding_window":
            mask_fn, block_fn = ref_masks.make_sliding_window_mask_fns(bq, bk, c["window"])
        elif c["kind"] == "document":
            mask_fn, block_fn = ref_masks.make_jagged_mask_fns(bq, bk, c["doc_lengths"])
        elif c["kind"] == "s2":
            mask_fn, block_fn = ref_masks.make_s2_mask_fns(bq, bk, c["window"], c["stride"])
        else:
            mask_fn, block_fn = ref_masks.place_holder(bq, bk)
        idx = np.arange(s)
        if c["kind"] == "none":
            dense = np.ones((s, s), bool)
        else:
            dense = np.asarray(mask_fn(idx, idx), bool)
        nq, nk = -(-s // bq), -(-s // bk)
        blocks = np.zeros((nq, nk), bool)
        for i in range(nq):
            for j in range(nk):
                blocks[i, j] = bool(block_fn(np.int64(i), np.int64(j)))
        out[f"mask/{name}/dense"] = np.packbits(dense, axis=-1)
        out[f"mask/{name}/blocks"] = blocks

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
