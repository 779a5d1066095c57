#!/usr/bin/env python
"""Benchmark of the flex-attention hot path (forward + delta preprocess + dQ + dK/dV) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload t|c1|c2|c3|c4|...] [--impl ours|reference]

One "step" = one forward and one backward pass of the hot path over one batch of synthetic input.
Prints ONE JSON line (rank 0).  The metric is causal-adjusted attention TFLOP/s = kept-pair FLOPs
(fwd 4*B*H*D*pairs + bwd 10*B*H*D*pairs) / time, whole job over all GPUs.

The headline workload is `t`: causal, bf16, B=4 H=32 S=8192 D=128, the shape the throughput target is quoted
on.  With N > 1 every rank runs that per-GPU workload on its own (batch x head) shard (weak scaling, no
collective on the data path; NCCL only for the barrier and the max-over-ranks time).  Further legs, each a key
of the same JSON line:

  workloads    the other benchmark configurations (c1 .. c4) and the score_mod sweep at the target shape, each
               timed as a CUDA-graph replay of the whole step
  kernels      every kernel of the path timed from a graph of back-to-back launches (no host latency inside)
  e2e          the same step through the host-buffer API, pinned host memory in and out, with the time of the
               copies alone next to it
  c5_sharded   ONE global problem (B=16 H=64 S=32768 D=128, causal) sharded by (batch x head) over the N ranks
               (strong scaling), with sampled output slices gathered over NCCL and verified by another rank
  cpu_baseline the CPU restatement of the reference's dense definitions on the host cores (rank 0, N = 1)

`--impl reference` times that CPU restatement alone (JAX, the reference's only runtime, is not installed).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import workloads  # noqa: E402  (document layouts, kept-pair counts; next to this file)

METRIC = "fwd+bwd attention TFLOP/s (causal-adjusted)"
NOMINAL_TFLOPS = 2250.0   # dense bf16, for context next to the measured peak

# Per-GPU workloads.  c1..c4 = the first four benchmark configurations; t = the S=8192, D=128 target point;
# t_* = the same shape with no mask and with each score_mod; c5 = the sharded long-sequence configuration
# (whole problem: --workload c5 runs it on one GPU, the c5_sharded leg splits it over the ranks).
WORKLOADS = {
    "c1": dict(B=1, H=4, S=512, D=64, seed=0, mask="causal", score="none", dtype="f32",
               desc="causal MHA fwd+bwd fp32 B=1 H=4 S=512 D=64 (BASELINE configs[0])"),
    "c2": dict(B=8, H=16, S=2048, D=128, seed=1, mask="causal", score="none",
               desc="causal MHA fwd+bwd bf16 B=8 H=16 S=2048 D=128 (BASELINE configs[1])"),
    "t": dict(B=4, H=32, S=8192, D=128, seed=5, mask="causal", score="none",
              desc="causal MHA fwd+bwd bf16 B=4 H=32 S=8192 D=128 (the S=8192, D=128 target point)"),
    "t_nomask": dict(B=4, H=32, S=8192, D=128, seed=5, mask="none", score="none",
                     desc="unmasked MHA fwd+bwd bf16 B=4 H=32 S=8192 D=128"),
    "t_alibi": dict(B=4, H=32, S=8192, D=128, seed=5, mask="causal", score="alibi",
                    desc="causal + ALiBi fwd+bwd bf16 B=4 H=32 S=8192 D=128"),
    "t_softcap": dict(B=4, H=32, S=8192, D=128, seed=5, mask="causal", score="softcap", cap=50.0,
                      desc="causal + tanh softcap(50) fwd+bwd bf16 B=4 H=32 S=8192 D=128"),
    "c3": dict(B=4, H=32, S=8192, D=128, seed=2, mask="sliding_window_causal", window=256, score="alibi",
               desc="sliding-window(256, causal) + ALiBi fwd+bwd bf16 B=4 H=32 S=8192 D=128 (BASELINE configs[2])"),
    "c4": dict(B=2, H=16, S=16384, D=128, seed=3, mask="document", score="softcap", cap=50.0,
               desc="document mask + tanh softcap(50) fwd+bwd bf16 B=2 H=16 S=16384 D=128 (BASELINE configs[3])"),
    "c5": dict(B=16, H=64, S=32768, D=128, seed=4, mask="causal", score="none",
               desc="causal MHA fwd+bwd bf16 B=16 H=64 S=32768 D=128 (BASELINE configs[4])"),
}
SUB_WORKLOADS = ("c1", "c2", "c3", "c4", "t_nomask", "t_alibi", "t_softcap")
E2E_CHUNK_HEADS = 8   # the host-buffer pipeline moves chunks of 8 heads of one batch row (67 MB per tensor at S=8192)

# dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel, from the ncu captures summarised under
# profiles/ (None where no capture of the current kernel exists).
NCU_TRAFFIC_BYTES = {"c2": {"fwd": 276.4e6, "dq": 369.1e6, "dkv": 380.4e6},
                     "t": {"fwd": 1064.7e6, "dq": 1862.1e6, "dkv": 1599.3e6}}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(tflops=float(d["bf16_tflops"]), tflops_sustained=float(d.get("bf16_tflops_sustained", 0)),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


def total_pairs(w, doc_ids=None):
    per_row = workloads.kept_pairs(w["mask"], w["S"], window=w.get("window", 0), stride=w.get("stride", 0),
                                   doc_ids=doc_ids)   # one entry per batch row for document masks, else one
    if len(per_row) == 1:
        return per_row[0] * w["B"] * w["H"]
    return sum(per_row) * w["H"]


def elt_bytes(w):
    return 4 if w.get("dtype") == "f32" else 2


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """nvidia-smi sampling in a child process.  Started well before the timed region (its start-up talks
    to the driver and would disturb the first launches otherwise); samples are kept only if their
    timestamp falls inside the window given to stop().  Query only: no setting of the GPU is touched."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, period_ms=20):
        self.proc, self.index, self.period_ms = None, index, period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        # block until the first sample arrives: nvidia-smi's start-up (driver/NVML initialisation) must be
        # over before anything is timed
        import select
        ready, _, _ = select.select([self.proc.stdout], [], [], 15.0)
        self.first = self.proc.stdout.readline() if ready else ""

    def stop(self, t_begin, t_end):
        import datetime
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        out = getattr(self, "first", "") + out
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = []
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), float(parts[3]),
                             [n for n, v in zip(names, parts[4:8]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if t_begin <= r[0] <= t_end]
        note = "samples inside the timed region"
        if not inside and rows:   # region shorter than the sampling period: take the nearest sample
            mid = 0.5 * (t_begin + t_end)
            inside = [min(rows, key=lambda r: abs(r[0] - mid))]
            note = "timed region shorter than the sampling period: nearest sample"
        if not inside:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        reasons = sorted({x for r in inside for x in r[4]})
        return dict(sm_mhz=float(np.median([r[1] for r in inside])), sm_max_mhz=float(max(r[2] for r in inside)),
                    power_w=float(np.median([r[3] for r in inside])), reasons=reasons, samples=len(inside),
                    note=note)


# ------------------------------------------------------------------------------------------ inputs
def make_device_inputs(w, rank, torch):
    """Synthetic q, k, v, do ~ N(0,1), generated on the device from the workload seed (+ rank)."""
    g = torch.Generator(device="cuda").manual_seed(w["seed"] * 1000 + rank)
    shape = (w["B"], w["H"], w["S"], w["D"])
    dt = torch.float32 if w.get("dtype") == "f32" else torch.bfloat16
    return [torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).to(dt) for _ in range(4)]


def make_mods(w, fa, rank):
    seg = None
    doc = None
    if w["mask"] == "causal":
        mf, bf = fa.masks.make_causal_mask_fns(128, 128)
    elif w["mask"] == "sliding_window_causal":
        mf, bf = fa.masks.make_sliding_window_mask_fns(128, 128, w["window"], causal=True)
    elif w["mask"] == "document":
        doc, _ = workloads.draw_documents(np.random.default_rng(w["seed"] * 1000 + rank), w["B"], w["S"])
        mf, bf, seg = None, None, doc
    else:
        mf, bf = fa.masks.place_holder(128, 128)
    sf = None
    if w["score"] == "alibi":
        sf = fa.scores.make_alibi_score_fn(fa.scores.alibi_slopes(w["H"]))
    elif w["score"] == "softcap":
        sf = fa.scores.make_softcap_score_fn(w["cap"])
    return mf, bf, sf, seg, doc


class HotPath:
    """fwd + preprocess + dq + dkv through the package's reference-named entry points."""

    def __init__(self, w, fa, torch, rank):
        self.fa, self.torch, self.w = fa, torch, w
        self.mf, self.bf, self.sf, seg, self.doc = make_mods(w, fa, rank)
        self.seg = None if seg is None else torch.from_numpy(seg).cuda()
        self.sm_scale = 1.0 / float(np.sqrt(w["D"]))

    def fwd(self, q, k, v):
        return self.fa._flex_attention_impl(q, k, v, None, self.seg, True, False, self.sm_scale, 1, 128, 128, 128,
                                            False, self.bf, self.mf, self.sf)

    def bwd(self, q, k, v, o, l, m, do):
        # delta, then dQ and dK/dV (the package launches the two gradient kernels on two streams)
        return self.fa.flex_attention_bwd(q, k, v, o, l, m, do, segment_ids=self.seg, sm_scale=self.sm_scale,
                                          mask_fns=None if self.mf is None else (self.mf, self.bf), score_fn=self.sf)

    def step(self, q, k, v, do):
        o, l, m = self.fwd(q, k, v)
        dq, dk, dv = self.bwd(q, k, v, o, l, m, do)
        return o, dq, dk, dv


def capture_step(hp, q, k, v, do, torch):
    """Two CUDA graphs (forward, backward) captured from exactly the entry-point calls of a step.  At ~1 ms per
    step the host cannot always keep the GPU fed through Python (shared host cores), so timed steps replay them."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        hp.step(q, k, v, do)                      # allocator / lazy-init warm-up on the capture stream
        g_fwd, g_bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_fwd, stream=side):
            o, l, m = hp.fwd(q, k, v)
        with torch.cuda.graph(g_bwd, stream=side, pool=g_fwd.pool()):
            out = hp.bwd(q, k, v, o, l, m, do)
    torch.cuda.current_stream().wait_stream(side)
    g_fwd.replay()
    g_bwd.replay()
    torch.cuda.synchronize()
    return g_fwd, g_bwd, (o, l, m) + tuple(out)


def time_replays(g_fwd, g_bwd, steps, torch):
    """Device time of `steps` replays: (total ms, mean fwd ms, mean bwd ms), CUDA events on the current stream."""
    e0 = torch.cuda.Event(enable_timing=True)
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    e0.record()
    for a, b in marks:
        g_fwd.replay()
        a.record()
        g_bwd.replay()
        b.record()
    torch.cuda.synchronize()
    fwd_ms, bwd_ms, prev = [], [], e0
    for a, b in marks:
        fwd_ms.append(prev.elapsed_time(a))
        bwd_ms.append(a.elapsed_time(b))
        prev = b
    return e0.elapsed_time(marks[-1][1]), float(np.mean(fwd_ms)), float(np.mean(bwd_ms))


def time_kernels(hp, q, k, v, do, torch, reps=20, rounds=3):
    """Device time per launch of each kernel of the path: a CUDA graph of `reps` back-to-back launches of that
    kernel alone, replayed `rounds` times between two events (first replay discarded), so that no host launch
    latency sits between the events."""
    fa = hp.fa
    o, l, m = hp.fwd(q, k, v)
    delta = fa.bwd_preprocess(o, do)
    calls = {
        "fwd": lambda: hp.fwd(q, k, v),
        "delta": lambda: fa.bwd_preprocess(o, do),
        "dq": lambda: fa.flex_attention_bwd_dq(q, k, v, None, hp.seg, l, m, o, do, delta, sm_scale=hp.sm_scale,
                                               score_fn=hp.sf, mask_fn=hp.mf, block_mask_fn=hp.bf),
        "dkv": lambda: fa.flash_attention_bwd_dkv(k, v, q, None, hp.seg, l, m, delta, do, sm_scale=hp.sm_scale,
                                                  score_fn=hp.sf, mask_fn=hp.mf, block_mask_fn=hp.bf),
    }
    out = {}
    side = torch.cuda.Stream()
    for name, fn in calls.items():
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(reps):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(rounds - 1):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / (reps * (rounds - 1))
        del g
    return out


def workload_record(name, fa, torch, rank, steps, peaks):
    """One sub-record of the JSON line: the whole step of workload `name`, replayed from CUDA graphs."""
    w = WORKLOADS[name]
    q, k, v, do = make_device_inputs(w, rank, torch)
    hp = HotPath(w, fa, torch, rank)
    pairs = total_pairs(w, hp.doc)
    for _ in range(3):
        hp.step(q, k, v, do)
    g_fwd, g_bwd, _ = capture_step(hp, q, k, v, do, torch)
    time_replays(g_fwd, g_bwd, 3, torch)
    total_ms, fwd_ms, bwd_ms = time_replays(g_fwd, g_bwd, steps, torch)
    f_fwd, f_bwd = 4.0 * w["D"] * pairs, 10.0 * w["D"] * pairs
    rows, eb = w["B"] * w["H"] * w["S"], elt_bytes(w)
    bytes_fwd = 4 * rows * w["D"] * eb + 2 * rows * 4
    bytes_bwd = 8 * rows * w["D"] * eb + 3 * rows * 4
    tf = lambda fl, ms: fl / (ms * 1e-3) / 1e12
    rec = {
        "workload": w["desc"], "dtype": w.get("dtype", "bf16"), "steps": steps, "ms_per_step": total_ms / steps,
        "tflops": tf(f_fwd + f_bwd, total_ms / steps),
        "fwd": {"ms": fwd_ms, "tflops": tf(f_fwd, fwd_ms), "frac_of_peak": tf(f_fwd, fwd_ms) / peaks["tflops"],
                "gbs": bytes_fwd / (fwd_ms * 1e-3) / 1e9, "frac_of_hbm_peak": bytes_fwd / (fwd_ms * 1e-3) / 1e9 / peaks["hbm"]},
        "bwd": {"ms": bwd_ms, "tflops": tf(f_bwd, bwd_ms), "frac_of_peak": tf(f_bwd, bwd_ms) / peaks["tflops"],
                "gbs": bytes_bwd / (bwd_ms * 1e-3) / 1e9, "frac_of_hbm_peak": bytes_bwd / (bwd_ms * 1e-3) / 1e9 / peaks["hbm"]},
    }
    del g_fwd, g_bwd, q, k, v, do, hp
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------ C5, sharded
def c5_slice_seed(b, h):
    """Seed of slice (b, h) of the global problem: the same on every world size, so every slice has the same
    inputs - and the deterministic kernels the same outputs - however the problem is sharded."""
    return 4_000_000 + b * 64 + h


def fill_slices(tensors, units, torch):
    """tensors: q, k, v, do as [1, n, S, D]; units: the global (batch*head) indices of the n slices."""
    for i, u in enumerate(units):
        g = torch.Generator(device="cuda").manual_seed(c5_slice_seed(u // 64, u % 64))
        for t in tensors:
            t[0, i].normal_(generator=g)


def slice_errors(got, ref, torch):
    """Error figures of one bf16 slice against a bf16-stored reference, under the parity rule of the test-suite:
    raw max-abs and max-rel, max-abs beyond the two bf16 store roundings (half a unit in the last place of the
    reference value each), and the flat max-abs over elements whose reference is below 4."""
    g, r = got.float(), ref.float()
    diff = (g - r).abs()
    _, e = torch.frexp(r.abs())
    half_ulp = torch.ldexp(torch.ones_like(r), e - 9)
    small = r.abs() < 4.0
    return {"max_abs": float(diff.max()), "max_rel": float(diff.max() / r.abs().max().clamp_min(1e-30)),
            "max_abs_excess": float((diff - 2.0 * half_ulp).max()),
            "max_abs_small": float(diff[small].max()) if bool(small.any()) else 0.0}


def run_c5_sharded(fa, torch, dist, world, rank, peaks, steps=2):
    """Strong scaling on ONE global problem: B=16 H=64 S=32768 D=128 causal, the (batch x head) index split into
    `world` contiguous shards with no collective on the data path.  Afterwards the first and the last slice of
    every rank's O, dQ, dK, dV are all-gathered over NCCL and each rank checks the slices of its NEIGHBOUR against
    the fp32 SIMT backend run on that slice alone, from inputs regenerated out of the slice's seed."""
    from flex_attention_tpu_b200 import sharding
    w = WORKLOADS["c5"]
    units_total = w["B"] * w["H"]
    need = 8 * (units_total // world) * w["S"] * w["D"] * 2 + (8 << 30)
    free, _ = torch.cuda.mem_get_info()
    if free < need:
        return {"skipped": f"needs {need >> 30} GiB of device memory per GPU, {free >> 30} GiB free"}
    lo, hi = sharding.shard_bounds(units_total, world, rank)
    n = hi - lo
    shape = (1, n, w["S"], w["D"])
    q, k, v, do = (torch.empty(shape, dtype=torch.bfloat16, device="cuda") for _ in range(4))
    fill_slices((q, k, v, do), range(lo, hi), torch)
    hp = HotPath(dict(w, B=1, H=n), fa, torch, rank)
    out = hp.step(q, k, v, do)          # warm-up (builds the mask map)
    del out
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        o, dq, dk, dv = hp.step(q, k, v, do)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    pairs = workloads.kept_pairs("causal", w["S"])[0] * units_total
    tflops = 14.0 * w["D"] * pairs / (ms * 1e-3) / 1e12

    # ---- verification gather (outside the timed region): first and last slice of every shard
    picks = [0, n - 1]
    names = ("o", "dq", "dk", "dv")
    mine = {nm: t[:, picks].contiguous() for nm, t in zip(names, (o, dq, dk, dv))}       # [1, 2, S, D]
    if world > 1:
        gathered = {nm: sharding.gather_batch_heads(t, world, 2) for nm, t in mine.items()}   # [world, 2, S, D]
    else:
        gathered = {nm: t.reshape(1, 2, w["S"], w["D"]) for nm, t in mine.items()}
    del o, dq, dk, dv, q, k, v, do
    torch.cuda.empty_cache()
    peer = (rank + 1) % world
    plo, phi = sharding.shard_bounds(units_total, world, peer)
    worst = {nm: 0.0 for nm in names}
    worst_excess = 0.0
    ok = True
    sums = {}
    for j, u in enumerate((plo, phi - 1)):
        sq, sk, sv, sdo = (torch.empty((1, 1, w["S"], w["D"]), dtype=torch.bfloat16, device="cuda") for _ in range(4))
        fill_slices((sq, sk, sv, sdo), [u], torch)
        hs = HotPath(dict(w, B=1, H=1), fa, torch, rank)
        so, sl_, sm_ = fa._flex_attention_impl(sq, sk, sv, None, None, True, False, hs.sm_scale, 1, 128, 128, 128, False,
                                               hs.bf, hs.mf, None, backend="simt")
        sdq, sdk, sdv = fa.flex_attention_bwd(sq, sk, sv, so, sl_, sm_, sdo, sm_scale=hs.sm_scale,
                                              mask_fns=(hs.mf, hs.bf), backend="simt")
        for nm, ref in zip(names, (so, sdq, sdk, sdv)):
            got = gathered[nm][peer, j]
            e = slice_errors(got, ref[0, 0], torch)
            worst[nm] = max(worst[nm], e["max_abs"])
            worst_excess = max(worst_excess, e["max_abs_excess"])
            ok = ok and e["max_abs_excess"] <= 2e-2 and e["max_abs_small"] <= 2e-2 and e["max_rel"] <= 1e-2
            # bit pattern checksum of the slice: identical on every world size if the sharding changes nothing
            sums[f"{nm}[{u}]"] = int(got.view(torch.int16).to(torch.int64).sum().item())
    stats = torch.tensor([0.0 if ok else 1.0, worst_excess] + [worst[nm] for nm in names], dtype=torch.float64, device="cuda")
    all_sums = [sums]
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        all_sums = [None] * world
        dist.all_gather_object(all_sums, sums)
    merged = {}
    for s in all_sums:
        merged.update(s)
    st = stats.tolist()
    return {
        "workload": w["desc"], "scaling": "strong", "units_per_gpu": n, "steps": steps, "ms_per_step": ms, "tflops": tflops,
        "frac_of_peak_per_gpu": tflops / world / peaks["tflops"],
        "verification": {"pass": st[0] == 0.0,
                         "what": "first and last (batch, head) slice of every rank's O, dQ, dK, dV, all-gathered over NCCL, "
                                 "checked by the next rank against the fp32 SIMT backend on inputs regenerated from the slice seed",
                         "slices": 2 * world, "max_abs": dict(zip(names, st[2:])), "max_abs_beyond_store_rounding": st[1],
                         "bit_checksums": {k_: merged[k_] for k_ in sorted(merged)}},
    }


# ------------------------------------------------------------------------------------------ CPU legs
def cpu_reference_sample(w, budget_s=15.0, max_slices=None):
    """Times the CPU restatement of mha_reference + mha_bwd_reference on (batch, head) slices of the
    workload, one slice per host thread, for about `budget_s` seconds.  Inputs are drawn before the clock
    starts.  Returns (TFLOP/s, cores, text, seconds per slice)."""
    from oracle import mha_reference_cpu as oracle
    try:
        from threadpoolctl import threadpool_limits
    except ImportError:  # pragma: no cover
        threadpool_limits = None
    cores = min(os.cpu_count() or 1, 32)
    S, D = w["S"], w["D"]
    rng = np.random.default_rng(w["seed"])
    doc = None
    if w["mask"] == "document":
        doc, _ = oracle.draw_documents(rng, 1, S)
    kw = dict(sm_scale=1.0 / np.sqrt(D), mask_kind=w["mask"], window=w.get("window"), doc_ids=doc,
              score_kind=w["score"], cap=w.get("cap"), alibi_slopes=oracle.alibi_slopes(1))
    pairs = oracle.kept_pairs(w["mask"], S, S, window=w.get("window"), doc_ids=doc)[0]
    # one input set per thread, drawn outside the timed region and reused by that thread's slices
    pool = [[np.random.default_rng(1000 + i).standard_normal((1, 1, S, D), dtype=np.float32) for _ in range(4)]
            for i in range(cores)]

    def one_slice(i):
        q, k, v, do = pool[i % cores]
        o, l, m = oracle.mha_reference(q, k, v, save_residuals=True, **kw)
        oracle.mha_bwd_reference(q, k, v, o, do, l, m, **kw)

    def run(n):
        t0 = time.perf_counter()
        with ThreadPoolExecutor(cores) as ex:
            list(ex.map(one_slice, range(n)))
        return time.perf_counter() - t0

    ctx = threadpool_limits(limits=1) if threadpool_limits else None
    try:
        t1 = run(cores)                       # one slice per thread: calibrates the sample size
        n = int(max(cores, min(max_slices or 10 ** 9, cores * max(1, round(budget_s / max(t1, 1e-3))))))
        t = run(n) if n > cores else t1
        n = n if n > cores else cores
    finally:
        if ctx is not None:
            ctx.__exit__(None, None, None)
    flops = 14.0 * D * pairs * n
    sample = (f"{n} independent (batch, head) slices of the workload's shape (the workload has {w['B'] * w['H']}), "
              f"fwd+bwd, {t:.1f} s on {cores} threads")
    return flops / t / 1e12, cores, sample, t / n


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step_budget = min(15.0, 150.0 / max(1, args.steps + args.warmup))
    vals, sample, cores = [], "", 1
    for it in range(args.warmup + args.steps):
        v, cores, sample, _ = cpu_reference_sample(w, budget_s=per_step_budget)
        if it >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"], "note": "CPU restatement of the reference's mha_reference / "
                   "mha_bwd_reference (JAX is not installed, so the reference itself cannot run)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ main arm
def run_ours(args, w):
    import torch
    import torch.distributed as dist
    import flex_attention_tpu_b200 as fa

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks = measured_peaks()
    q, k, v, do = make_device_inputs(w, rank, torch)
    hp = HotPath(w, fa, torch, rank)
    pairs = total_pairs(w, hp.doc)
    flops_fwd = 4.0 * w["D"] * pairs
    flops_bwd = 10.0 * w["D"] * pairs

    # ---- device-resident timing: W warm-up steps, K timed steps, CUDA events, max over ranks
    sampler = ClockSampler(local_rank)
    sampler.start()
    hp.step(q, k, v, do)
    torch.cuda.synchronize()
    g_fwd = g_bwd = None
    if not args.no_graph:
        g_fwd, g_bwd, _ = capture_step(hp, q, k, v, do, torch)
    for _ in range(args.warmup):
        if g_fwd is not None:
            g_fwd.replay()
            g_bwd.replay()
        else:
            hp.step(q, k, v, do)
    barrier()
    t_begin = time.time()
    if g_fwd is not None:
        total_ms, fwd_ms, bwd_ms = time_replays(g_fwd, g_bwd, args.steps, torch)
    else:
        e0 = torch.cuda.Event(enable_timing=True)
        marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        e0.record()
        for a, b_ in marks:
            o, l, m = hp.fwd(q, k, v)
            a.record()
            hp.bwd(q, k, v, o, l, m, do)
            b_.record()
        torch.cuda.synchronize()
        total_ms = e0.elapsed_time(marks[-1][1])
        fwd_ms = float(np.mean([(e0 if i == 0 else marks[i - 1][1]).elapsed_time(marks[i][0]) for i in range(args.steps)]))
        bwd_ms = float(np.mean([a.elapsed_time(b_) for a, b_ in marks]))
    barrier()
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end)
    total_ms = max_over_ranks(total_ms)
    ms_step = total_ms / args.steps
    value = world * (flops_fwd + flops_bwd) / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public entry points with HOST buffers (pinned): H2D of q,k,v,do and
    # D2H of o,dq,dk,dv inside the timed region, every step
    e2e = None
    if not args.skip_e2e:
        from flex_attention_tpu_b200 import host_api
        host_in = [t.cpu().pin_memory() for t in (q, k, v, do)]
        host_out = [torch.empty_like(t).pin_memory() for t in host_in]
        io_bytes = sum(t.numel() * t.element_size() for t in host_in)

        def e2e_step():
            # chunks of the batch flow through copy-in, compute and copy-out streams so that the PCIe transfers
            # overlap the kernels and each other
            host_api.fwd_bwd_from_host(*host_in, sm_scale=hp.sm_scale, mask_fn=hp.mf, block_mask_fn=hp.bf, score_fn=hp.sf,
                                       segment_ids=hp.seg, out=host_out, chunk_batch=1, chunk_heads=E2E_CHUNK_HEADS)

        def copy_only_step():
            # the same bytes over the same pinned buffers, both directions at once, no kernels: the ceiling of e2e
            s_in, s_out = copy_streams
            for b0 in range(w["B"]):
                for h0 in range(0, w["H"], ch):
                    with torch.cuda.stream(s_in):
                        for d_, h_ in zip(stage_in, host_in):
                            d_.copy_(h_[b0:b0 + 1, h0:h0 + ch], non_blocking=True)
                    with torch.cuda.stream(s_out):
                        for h_, d_ in zip(host_out, stage_out):
                            h_[b0:b0 + 1, h0:h0 + ch].copy_(d_, non_blocking=True)
            for s in copy_streams:
                torch.cuda.current_stream().wait_stream(s)
            torch.cuda.current_stream().synchronize()

        def timed(fn, n):
            barrier()
            t0 = time.perf_counter()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(n):
                fn()
            g1.record()
            barrier()
            return max_over_ranks(g0.elapsed_time(g1)) / n, (time.perf_counter() - t0) * 1e3 / n

        e2e_steps = max(1, min(args.steps, 10))
        for _ in range(3):          # pinned-buffer paging and the side streams' allocator pools settle
            e2e_step()
        e2e_ms, e2e_wall_ms = timed(e2e_step, e2e_steps)
        copy_streams = (torch.cuda.Stream(), torch.cuda.Stream())
        ch = min(E2E_CHUNK_HEADS, w["H"]) if w["H"] % min(E2E_CHUNK_HEADS, w["H"]) == 0 else w["H"]
        stage_in = [torch.empty((1, ch, *t.shape[2:]), dtype=t.dtype, device="cuda") for t in host_in]
        stage_out = [torch.empty_like(t) for t in stage_in]
        copy_only_step()
        copy_ms, _ = timed(copy_only_step, e2e_steps)
        e2e = {"value": world * (flops_fwd + flops_bwd) / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes, "ms_per_step": e2e_ms,
               "wall_ms_per_step": e2e_wall_ms, "steps": e2e_steps, "copy_only_ms_per_step": copy_ms,
               "frac_of_copy_ceiling": copy_ms / e2e_ms,
               "copy_only_gbs_per_gpu_each_way": io_bytes / (copy_ms * 1e-3) / 1e9}
        del host_in, host_out, stage_in, stage_out

    # ---- per-kernel times and the other workloads (rank 0; outside every timed region)
    kt = subs = None
    if rank == 0:
        kt = time_kernels(hp, q, k, v, do, torch)
        if not args.skip_workloads:
            del g_fwd, g_bwd
            subs = {}
            for name in SUB_WORKLOADS:
                if name != args.workload:
                    subs[name] = workload_record(name, fa, torch, rank, 20, peaks)
    del q, k, v, do
    g_fwd = g_bwd = None
    torch.cuda.empty_cache()

    # ---- one global problem sharded over the ranks, with its verification gather
    c5 = None
    if not args.skip_c5:
        c5 = run_c5_sharded(fa, torch, dist, world, rank, peaks)

    if rank == 0:
        # executed-algorithmic FLOPs of each kernel: GEMMs it has to compute x kept pairs
        kflops = {"fwd": 4.0, "dq": 6.0, "dkv": 8.0}
        dom = max(("fwd", "dq", "dkv"), key=lambda n: kt[n])
        ach = kflops[dom] * w["D"] * pairs / (kt[dom] * 1e-3) / 1e12
        rows = w["B"] * w["H"] * w["S"]
        delta_bytes = 2 * rows * w["D"] * elt_bytes(w) + rows * 4
        peak_note = f"bf16_tflops (burst) of {peaks['source']} peaks"
        roofline = {"kernel": f"{dom}_sm100_kernel", "bound": "tensor", "achieved": ach, "peak": peaks["tflops"],
                    "unit": "TFLOP/s", "frac": ach / peaks["tflops"], "traffic": (NCU_TRAFFIC_BYTES.get(args.workload) or {}).get(dom),
                    "peak_source": peak_note, "ms_per_launch": kt[dom], "frac_of_nominal": ach / NOMINAL_TFLOPS}
        per_kernel = {n: {"ms": kt[n], "tflops": kflops[n] * w["D"] * pairs / (kt[n] * 1e-3) / 1e12,
                          "frac_of_peak": kflops[n] * w["D"] * pairs / (kt[n] * 1e-3) / 1e12 / peaks["tflops"]}
                      for n in ("fwd", "dq", "dkv")}
        per_kernel["delta"] = {"ms": kt["delta"], "gbs": delta_bytes / (kt["delta"] * 1e-3) / 1e9,
                               "frac_of_hbm_peak": delta_bytes / (kt["delta"] * 1e-3) / 1e9 / peaks["hbm"]}
        per_kernel["note"] = ("each kernel alone, from a graph of 20 back-to-back launches; inside a step dQ and dK/dV "
                              "overlap on two streams, so their sum exceeds the step's backward time")
        tf_fwd, tf_bwd = flops_fwd / (fwd_ms * 1e-3) / 1e12, flops_bwd / (bwd_ms * 1e-3) / 1e12
        # which regime the timed region ran in, from the clocks sampled inside it
        regime = None
        if clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
            regime = ("burst clocks" if clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"] else
                      "power-capped clocks (median SM %.0f of %.0f MHz): the sustained peak %.0f TFLOP/s is the like-for-like "
                      "denominator; fractions below still divide by the burst peak" %
                      (clocks["sm_mhz"], clocks["sm_max_mhz"], peaks["tflops_sustained"]))
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if w.get("dtype") == "f32" else "bf16", "data": "synthetic",
            "config": {"workload": w["desc"], "global_batch": w["B"] * world, "sharding": "batch x head, no collective",
                       "l2": "inputs (q,k,v,do) and outputs exceed the 126 MB L2; no flush needed",
                       "cuda_graph": not args.no_graph},
            "clocks": dict(clocks, regime=regime),
            "gpu_launches": 4 * args.steps,
            "roofline": roofline,
            "frac_of_peak": value / world / peaks["tflops"], "peak_tflops": peaks["tflops"], "peak_source": peak_note,
            "fwd": {"ms": fwd_ms, "tflops": tf_fwd, "frac_of_peak": tf_fwd / peaks["tflops"],
                    "frac_of_sustained_peak": tf_fwd / peaks["tflops_sustained"], "frac_of_nominal": tf_fwd / NOMINAL_TFLOPS},
            "bwd": {"ms": bwd_ms, "tflops": tf_bwd, "frac_of_peak": tf_bwd / peaks["tflops"],
                    "frac_of_sustained_peak": tf_bwd / peaks["tflops_sustained"], "frac_of_nominal": tf_bwd / NOMINAL_TFLOPS},
            "kernels": per_kernel,
        }
        if e2e is not None:
            line["e2e"] = e2e
        if subs:
            line["workloads"] = subs
        if c5 is not None:
            line["c5_sharded"] = c5
        if world == 1 and not args.skip_cpu_baseline:
            cpu_v, cores, sample, _ = cpu_reference_sample(w, budget_s=12.0)
            line["cpu_baseline"] = {"value": cpu_v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="t", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="time plain entry-point calls instead of CUDA-graph replays")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="omit the cpu_baseline leg (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--skip-workloads", action="store_true", help="omit the sub-records of the other workloads")
    ap.add_argument("--skip-c5", action="store_true", help="omit the sharded S=32768 leg and its verification gather")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
