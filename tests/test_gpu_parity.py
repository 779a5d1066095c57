"""Parity of the CUDA hot path (through the reference-named Python entry points and the C ABI) with
(1) the committed fixtures produced by the reference's own mha_reference.py and (2) the CPU oracle on
seeded inputs, for every mask kind x score kind, both dtypes, both backends, ragged sizes."""
import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from golden_map import oracle_kwargs
from helpers import assert_close, check_output, errors, make_qkvdo, oracle_hot_path, run_hot_path
from oracle import mha_reference_cpu as oracle

pytestmark = pytest.mark.gpu


def _fa():
    import flex_attention_tpu_b200 as fa
    return fa


@pytest.mark.parametrize("name", sorted(CASES))
def test_float32_against_reference_vectors(name, golden):
    """fp32 inputs, CUDA-core kernels, against the vectors the reference's mha_reference.py produced."""
    fa = _fa()
    c = CASES[name]
    kw = oracle_kwargs(c)
    q, k, v, do = (torch.from_numpy(a).cuda() for a in make_inputs(c))
    got = run_hot_path(fa, q, k, v, do, sm_scale=kw["sm_scale"], mask_kind=kw.get("mask_kind", "none"),
                       score_kind=kw.get("score_kind", "none"), window=kw.get("window", 0), stride=kw.get("stride", 0),
                       doc_ids=kw.get("doc_ids"), cap=kw.get("cap", 0.0), slopes=kw.get("alibi_slopes"))
    want = {n: golden[f"{name}/{n}"] for n in ("o", "l", "m")}
    names = ["o"]
    if not c.get("softcap"):
        want.update({n: golden[f"{name}/{n}"] for n in ("dq", "dk", "dv")})
        names += ["dq", "dk", "dv"]
    assert_close(got, want, torch.float32, names=names, what=name)


MASKS = {
    "none": dict(),
    "causal": dict(),
    "sliding_window": dict(window=150),
    "sliding_window_causal": dict(window=200),
    "document": dict(),
    "s2": dict(window=96, stride=32),
}


def _case(mask_kind, score_kind, dtype, B, H, Sq, Sk, D, seed, backend):
    fa = _fa()
    (q, k, v, do), host = make_qkvdo((B, H, Sq, D), (B, H, Sk, D), seed, dtype)
    kw = dict(MASKS[mask_kind])
    doc = None
    if mask_kind == "document":
        doc, _ = oracle.draw_documents(np.random.default_rng(seed), B, max(Sq, Sk), lo=60, hi=300)
    slopes = oracle.alibi_slopes(H) if score_kind == "alibi" else None
    cap = 4.0 if score_kind == "softcap" else None
    sm_scale = 1.0 / np.sqrt(D)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    got = run_hot_path(fa, q, k, v, do, sm_scale=sm_scale, mask_kind=mask_kind, score_kind=score_kind,
                       backend=backend, window=kw.get("window", 0), stride=kw.get("stride", 0), doc_ids=doc,
                       cap=cap or 0.0, slopes=slopes, status=status)
    assert status.tolist() == [0, 0, 0, 0], f"device-side wait gave up: {status.tolist()}"
    want = oracle_hot_path(*host, sm_scale=sm_scale, mask_kind=mask_kind, score_kind=score_kind,
                           window=kw.get("window"), stride=kw.get("stride"), doc_ids=doc, cap=cap, slopes=slopes)
    e = errors(got["delta"], want["delta"])   # delta is f32 but built from the stored (bf16-rounded) o
    assert e["max_rel"] <= (1e-4 if dtype == torch.float32 else 1e-2), f"delta {e}"
    return assert_close(got, want, dtype, what=f"{mask_kind}/{score_kind}/{backend}/D{D}")


def test_baseline_config_1_float32():
    """The first benchmark configuration exactly as stated: causal MHA fwd+bwd, fp32, B=1, H=4, S=512, D=64,
    q, k, v, dO i.i.d. N(0,1) from seed 0, scale 1/sqrt(D); O, dQ, dK, dV against the CPU oracle, max-abs <= 2e-3."""
    _case("causal", "none", torch.float32, 1, 4, 512, 512, 64, 0, "auto")


@pytest.mark.parametrize("score_kind", ["none", "alibi", "softcap"])
@pytest.mark.parametrize("mask_kind", sorted(MASKS))
def test_simt_float32(mask_kind, score_kind):
    _case(mask_kind, score_kind, torch.float32, 2, 2, 333, 333, 64, 101, "auto")


@pytest.mark.parametrize("D", [32, 128])
def test_simt_float32_head_dims_and_rectangular(D):
    _case("none", "none", torch.float32, 1, 2, 200, 456, D, 102, "auto")
    _case("causal", "softcap", torch.float32, 1, 2, 456, 456, D, 103, "simt")


@pytest.mark.parametrize("score_kind", ["none", "alibi", "softcap"])
@pytest.mark.parametrize("mask_kind", sorted(MASKS))
def test_simt_bfloat16(mask_kind, score_kind):
    _case(mask_kind, score_kind, torch.bfloat16, 1, 2, 300, 300, 128, 104, "simt")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("score_kind", ["none", "alibi", "softcap"])
@pytest.mark.parametrize("mask_kind", sorted(MASKS))
def test_tensor_core_bfloat16(mask_kind, score_kind, D):
    """The tcgen05 kernels: every mask x score functor, both head dims, ragged sequence (not a tile multiple)."""
    _case(mask_kind, score_kind, torch.bfloat16, 2, 2, 777, 777, D, 105 + D, "tcgen05")


@pytest.mark.parametrize("Sq,Sk", [(128, 128), (100, 100), (256, 1024), (1000, 384), (129, 257), (300, 2000)])
def test_tensor_core_shapes(Sq, Sk):
    _case("none", "none", torch.bfloat16, 1, 3, Sq, Sk, 128, 300 + Sq, "tcgen05")
    if Sq == Sk:
        _case("causal", "none", torch.bfloat16, 1, 3, Sq, Sk, 128, 301 + Sq, "tcgen05")


def test_tensor_core_is_deterministic():
    fa = _fa()
    (q, k, v, do), _ = make_qkvdo((1, 4, 1024, 128), (1, 4, 1024, 128), 9, torch.bfloat16)
    a = run_hot_path(fa, q, k, v, do, sm_scale=0.088, mask_kind="causal", backend="tcgen05")
    b = run_hot_path(fa, q, k, v, do, sm_scale=0.088, mask_kind="causal", backend="tcgen05")
    for n in ("o", "l", "m", "dq", "dk", "dv"):
        assert torch.equal(a[n], b[n]), n


def test_tensor_core_matches_simt_on_long_rows():
    """Longer rows than the oracle cases: the two GPU backends must agree (SIMT is the fp32-accurate one)."""
    fa = _fa()
    (q, k, v, do), _ = make_qkvdo((1, 2, 4096, 128), (1, 2, 4096, 128), 10, torch.bfloat16)
    sm = 1.0 / np.sqrt(128)
    a = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", backend="tcgen05")
    b = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", backend="simt")
    for n in ("o", "dq", "dk", "dv"):
        check_output("tcgen05 vs simt", n, a[n], b[n], torch.bfloat16, roundings=2)   # both sides stored in bf16


@pytest.mark.parametrize("S", [128, 256, 384])
def test_persistent_forward_with_many_short_items(S):
    """The persistent forward walks several work items per CTA as one kv-tile stream, with Q K^T running three tiles
    (here: up to three ITEMS) ahead of the softmax.  Many one- to three-tile items per CTA exercise every item
    boundary hazard: Q stage reuse, the first P V of an item after the previous item's epilogue, the end of the list."""
    fa = _fa()
    (q, k, v, do), _ = make_qkvdo((5, 96, S, 64), (5, 96, S, 64), 600 + S, torch.bfloat16)
    sm = 0.125
    a = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", backend="tcgen05")
    b = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", backend="simt")
    for n in ("o", "dq", "dk", "dv"):
        check_output("tcgen05 vs simt", n, a[n], b[n], torch.bfloat16, roundings=2)   # both sides stored in bf16
    assert float((a["l"] / b["l"] - 1).abs().max()) <= 2e-2


def test_persistent_forward_rectangular_with_many_items():
    """Sq != Sk, no mask, several items per CTA (every item has the same five kv tiles)."""
    fa = _fa()
    (q, k, v, do), _ = make_qkvdo((4, 64, 256, 128), (4, 64, 640, 128), 611, torch.bfloat16)
    a = run_hot_path(fa, q, k, v, do, sm_scale=0.09, mask_kind="none", backend="tcgen05")
    b = run_hot_path(fa, q, k, v, do, sm_scale=0.09, mask_kind="none", backend="simt")
    for n in ("o", "dq", "dk", "dv"):
        check_output("tcgen05 vs simt", n, a[n], b[n], torch.bfloat16, roundings=2)   # both sides stored in bf16


@pytest.mark.parametrize("mask_kind,score_kind", [("document", "softcap"), ("sliding_window_causal", "alibi"),
                                                   ("s2", "none"), ("sliding_window", "none")])
def test_persistent_kernels_every_mask_with_many_items(mask_kind, score_kind):
    """Several work items per CTA (the persistent forward and dQ kernels walk them as one stream) under every mask
    family: item lengths differ from item to item, partial tiles sit at different places, document ids change with
    the batch row."""
    _case(mask_kind, score_kind, torch.bfloat16, 4, 48, 500, 500, 128, 900 + len(mask_kind), "tcgen05")


def test_error_is_operand_and_store_rounding():
    """Where the bf16 error of the tensor-core path comes from.  dV = P^T dO is modelled on the CPU with exactly the
    two roundings the kernel makes - the probabilities packed to bf16 the way the kernel packs them (pre-scaled by
    1 + 2^-9, then truncated), the result stored in bf16 - and everything else exact.  The GPU's error against the
    oracle must be the model's error: same size, and the same pattern (the two error vectors correlate).
    (Case: no mask + ALiBi at D = 128, the comparison with the largest dV error of the suite.)"""
    fa = _fa()
    B, H, S, D = 2, 2, 777, 128
    (q, k, v, do), host = make_qkvdo((B, H, S, D), (B, H, S, D), 105 + D, torch.bfloat16)
    slopes = oracle.alibi_slopes(H)
    sm = 1.0 / np.sqrt(D)
    got = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="none", score_kind="alibi", backend="tcgen05", slopes=slopes)
    qh, kh, vh, doh = host
    kw = dict(sm_scale=sm, mask_kind="none", score_kind="alibi", alibi_slopes=slopes)
    o, l, m = oracle.mha_reference(qh, kh, vh, save_residuals=True, **kw)
    _, _, dv = oracle.mha_bwd_reference(qh, kh, vh, o, doh, l, m, **kw)
    bf16 = lambda x: torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).float().numpy()
    model = np.empty_like(dv)
    i, j = np.arange(S)[:, None], np.arange(S)[None, :]
    for b in range(B):
        for h in range(H):
            t = (qh[b, h] @ kh[b, h].T) * np.float32(sm) - slopes[h] * (i - j).astype(np.float32)
            p = np.exp(t - m[b, h][:, None]) / l[b, h][:, None]
            packed = ((p * np.float32(1.001953125)).astype(np.float32).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
            model[b, h] = bf16(packed.T @ doh[b, h])
    gpu = got["dv"].float().cpu().numpy()
    e_gpu, e_model = np.abs(gpu - dv).max(), np.abs(model - dv).max()
    print("parity", {"case": "error model dv", "gpu_max_abs": float(e_gpu), "model_max_abs": float(e_model)})
    assert abs(e_gpu - e_model) <= 0.1 * e_model, (e_gpu, e_model)
    # ... and the same errors, element by element: the GPU accumulates in another order and uses ex2.approx, which
    # flips a rounding here and there, but its error vector is the model's (correlation close to one)
    eg, em = (gpu - dv).ravel().astype(np.float64), (model - dv).ravel().astype(np.float64)
    corr = float(np.dot(eg, em) / (np.linalg.norm(eg) * np.linalg.norm(em)))
    print("parity", {"case": "error model dv", "error_correlation": corr})
    assert corr >= 0.7, corr


@pytest.mark.parametrize("ids", ["repeating", "descending", "one_row_unsorted"])
@pytest.mark.parametrize("score_kind,D", [("none", 128), ("softcap", 64)])
def test_document_ids_need_not_be_sorted(ids, score_kind, D):
    """The document mask is defined by EQUAL ids.  When the ids of a batch row never decrease the kernels mask
    partial tiles from the bounds of each position's run of equal ids (computed once with the mask map); otherwise
    an id may come back after another one, a row's kept keys are no interval, and the kernels compare ids per
    element.  Both forms, and a batch that mixes them, against the oracle."""
    fa = _fa()
    B, H, S = 2, 2, 700
    pos = np.arange(S)
    if ids == "repeating":
        doc = np.stack([(pos // 90) % 3, (pos // 130) % 2]).astype(np.int32)            # ids come back
    elif ids == "descending":
        doc = np.stack([7 - pos // 100, 9 - pos // 64]).astype(np.int32)                # contiguous runs, decreasing ids
    else:
        doc = np.stack([pos // 150, (pos // 90) % 3]).astype(np.int32)                  # row 0 sorted, row 1 not
    (q, k, v, do), host = make_qkvdo((B, H, S, D), (B, H, S, D), 321, torch.bfloat16)
    cap = 4.0 if score_kind == "softcap" else None
    sm_scale = 1.0 / np.sqrt(D)
    for fwd_backend in ("tcgen05",):
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        got = run_hot_path(fa, q, k, v, do, sm_scale=sm_scale, mask_kind="document", score_kind=score_kind,
                           backend=fwd_backend, doc_ids=doc, cap=cap or 0.0, status=status)
        assert status.tolist() == [0, 0, 0, 0], status.tolist()
        want = oracle_hot_path(*host, sm_scale=sm_scale, mask_kind="document", score_kind=score_kind, doc_ids=doc, cap=cap)
        assert_close(got, want, torch.bfloat16, what=f"document ids {ids}/{score_kind}/D{D}")
