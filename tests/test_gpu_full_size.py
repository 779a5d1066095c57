"""The hot path at the benchmark configurations' full sizes, where the CPU oracle cannot cover the whole
tensor.  Checked through properties that hold at any size, plus exact comparisons on sampled (batch, head)
slices:

  * <dO, O> = <dV, V> per slice: O = P V is linear in V, so sum_i delta_i = <P^T dO, V>.
  * <dQ, Q> = <dK, K> per slice: the scaled score depends on q and k only through q.k, so both sides equal
    sum_ij ds_ij s_ij.  Holds for every mask and score functor of the build.
  * l >= 1 (the row maximum contributes exp(0)), m finite, |O| <= max|V| (rows of P sum to one).
  * sampled slices, in EVERY configuration: the tcgen05 result of one slice (b, h) taken out of the full launch
    against the CPU oracle run on that slice (row-blocked, seconds at S = 8192, about a minute at S = 32768), and
    of two more slices (first, last) against the fp32 SIMT backend run on the slice alone (itself checked against
    the oracle at small sizes).

Inputs are drawn on the device (seeded) because a host draw of these sizes takes longer than the kernels."""
import numpy as np
import pytest
import torch

import workloads

from helpers import check_output, oracle_hot_path, run_hot_path

pytestmark = pytest.mark.gpu

CONFIGS = {
    # name: batch, heads, seq, head_dim, mask, score, extra
    "c2": dict(B=8, H=16, S=2048, D=128, mask="causal", score="none"),
    "c3": dict(B=4, H=32, S=8192, D=128, mask="sliding_window_causal", score="alibi", window=256),
    "c4": dict(B=2, H=16, S=16384, D=128, mask="document", score="softcap", cap=50.0),
    "t": dict(B=4, H=32, S=8192, D=128, mask="causal", score="none"),
    # the largest configuration: 2^32 elements per tensor, so every offset that is not 64-bit shows up here
    "c5": dict(B=16, H=64, S=32768, D=128, mask="causal", score="none"),
    # every score functor (and no mask at all) at the S = 8192, D = 128 target shape
    "t_alibi": dict(B=1, H=8, S=8192, D=128, mask="causal", score="alibi"),
    "t_softcap": dict(B=1, H=8, S=8192, D=128, mask="causal", score="softcap", cap=50.0),
    "t_nomask": dict(B=1, H=8, S=8192, D=128, mask="none", score="none"),
}


def _fa():
    import flex_attention_tpu_b200 as fa
    return fa


def _inputs(cfg, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    shape = (cfg["B"], cfg["H"], cfg["S"], cfg["D"])
    return [torch.randn(shape, generator=g, device="cuda", dtype=torch.bfloat16) for _ in range(4)]


def _mods(cfg, seed):
    fa = _fa()
    kw = dict(mask_kind=cfg["mask"], score_kind=cfg["score"], window=cfg.get("window", 0), cap=cfg.get("cap", 0.0))
    if cfg["mask"] == "document":
        ids, _ = workloads.draw_documents(np.random.default_rng(seed), cfg["B"], cfg["S"])
        kw["doc_ids"] = ids
    if cfg["score"] == "alibi":
        kw["slopes"] = (2.0 ** (-8.0 * (np.arange(cfg["H"]) + 1) / cfg["H"])).astype(np.float32)
    return kw


def _slice_kw(kw, b, h):
    s = dict(kw)
    if s.get("doc_ids") is not None:
        s["doc_ids"] = s["doc_ids"][b:b + 1]
    if s.get("slopes") is not None:
        s["slopes"] = s["slopes"][h:h + 1]
    return s


def _dot_per_slice(a, b):
    """<a, b> per (batch, head) in f64, one batch row at a time to bound the temporaries."""
    out = torch.empty(a.shape[:2], dtype=torch.float64, device=a.device)
    for i in range(a.shape[0]):
        for j0 in range(0, a.shape[1], 8):
            out[i, j0:j0 + 8] = (a[i, j0:j0 + 8].double() * b[i, j0:j0 + 8].double()).sum(dim=(-1, -2))
    return out


def _abs_dot_per_slice(a, b):
    out = torch.empty(a.shape[:2], dtype=torch.float64, device=a.device)
    for i in range(a.shape[0]):
        for j0 in range(0, a.shape[1], 8):
            out[i, j0:j0 + 8] = (a[i, j0:j0 + 8].double() * b[i, j0:j0 + 8].double()).abs().sum(dim=(-1, -2))
    return out


def _need_memory(cfg):
    n = cfg["B"] * cfg["H"] * cfg["S"] * cfg["D"] * 2
    need = 8 * n + 4 * n // 8 + (6 << 30)     # 8 bf16 tensors, the f64 chunks of the reductions, slack
    free, _ = torch.cuda.mem_get_info()
    if free < need:
        pytest.skip(f"needs {need >> 30} GiB of device memory, {free >> 30} GiB free")


@pytest.mark.parametrize("name", ["c2", "c3", "c4", "t", "c5", "t_alibi", "t_softcap", "t_nomask"])
def test_full_size_properties_and_sampled_slices(name):
    fa, cfg = _fa(), CONFIGS[name]
    _need_memory(cfg)
    seed = 40 + sorted(CONFIGS).index(name)
    q, k, v, do = _inputs(cfg, seed)
    kw = _mods(cfg, seed)
    sm = 1.0 / np.sqrt(cfg["D"])
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    r = run_hot_path(fa, q, k, v, do, sm_scale=sm, backend="tcgen05", status=status, **kw)
    assert int(status[0]) == 0, status.tolist()

    # ---- size-independent properties, per (batch, head) slice
    for n in ("o", "dq", "dk", "dv", "l", "m", "delta"):
        assert bool(torch.isfinite(r[n]).all()), n
    assert float(r["l"].min()) >= 0.995
    assert float(r["o"].abs().max()) <= float(v.abs().max()) * 1.01
    lhs, rhs = r["delta"].double().sum(dim=-1), _dot_per_slice(r["dv"], v)
    scale = _abs_dot_per_slice(r["dv"], v)
    gap = ((lhs - rhs).abs() / scale).max().item()
    assert gap <= 2e-3, f"<dO,O> vs <dV,V>: {gap:.3e}"
    lhs, rhs = _dot_per_slice(r["dq"], q), _dot_per_slice(r["dk"], k)
    scale = 0.5 * (_abs_dot_per_slice(r["dq"], q) + _abs_dot_per_slice(r["dk"], k))
    gap = ((lhs - rhs).abs() / scale).max().item()
    assert gap <= 2e-3, f"<dQ,Q> vs <dK,K>: {gap:.3e}"

    # ---- sampled slices: one in the middle against the CPU oracle, first and last against the SIMT backend
    B, H = cfg["B"], cfg["H"]
    for (b, h, against) in [(B // 2, H // 3, "oracle"), (0, 0, "simt"), (B - 1, H - 1, "simt")]:
        sl = lambda t: t[b:b + 1, h:h + 1]
        skw = _slice_kw(kw, b, h)
        case = f"{name} slice ({b},{h}) tcgen05 vs {against}"
        if against == "oracle":
            host = [sl(t).float().cpu().numpy() for t in (q, k, v, do)]
            ref = oracle_hot_path(*host, sm_scale=sm, mask_kind=skw["mask_kind"], score_kind=skw["score_kind"],
                                  window=skw.get("window") or None, cap=skw.get("cap") or None,
                                  doc_ids=skw.get("doc_ids"), slopes=skw.get("slopes"))
            ref = {n: torch.from_numpy(np.ascontiguousarray(x)) for n, x in ref.items()}
            roundings = 1
        else:
            ref = run_hot_path(fa, sl(q), sl(k), sl(v), sl(do), sm_scale=sm, backend="simt", **skw)
            roundings = 2     # both sides stored in bf16
        for n in ("o", "dq", "dk", "dv"):
            check_output(case, n, sl(r[n]), ref[n], torch.bfloat16, roundings=roundings)
        assert float((sl(r["m"]).cpu() - ref["m"].cpu()).abs().max()) <= 2e-2, case
        assert float((sl(r["l"]).cpu() / ref["l"].cpu() - 1).abs().max()) <= 2e-2, case
    del q, k, v, do, r
    torch.cuda.empty_cache()
