"""The (batch x head) sharding logic on CPU with world_size 2 (gloo): shard -> per-rank work -> gather must
reproduce the unsharded result.  The per-rank work is the CPU oracle here; the GPU kernels take its place in
bench.py --gpus N."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flex_attention_tpu_b200 import sharding
        from oracle import mha_reference_cpu as oracle
        B, H, S, D = 2, 3, 40, 8          # 6 units over 2 ranks; also 5 units (uneven) below
        rng = np.random.default_rng(0)
        q, k, v = (torch.from_numpy(rng.standard_normal((B, H, S, D), dtype=np.float32)) for _ in range(3))
        full = oracle.mha_reference(q.numpy(), k.numpy(), v.numpy(), sm_scale=0.3, mask_kind="causal")
        qs, ks, vs = (sharding.shard_batch_heads(t, world, rank) for t in (q, k, v))
        mine = oracle.mha_reference(qs.numpy(), ks.numpy(), vs.numpy(), sm_scale=0.3, mask_kind="causal")
        got = sharding.gather_batch_heads(torch.from_numpy(mine), B, H)
        ok = np.allclose(got.numpy(), full, atol=1e-6)
        # uneven split: 5 units
        t = torch.arange(1 * 5 * 4, dtype=torch.float32).reshape(1, 5, 4)
        sh = sharding.shard_batch_heads(t, world, rank)
        ok = ok and torch.equal(sharding.gather_batch_heads(sh, 1, 5), t)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    from flex_attention_tpu_b200.sharding import shard_bounds
    for units in (1, 5, 128, 1024):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(units, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == units
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_shard_gather_roundtrip_world2():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, _free_port_once(), ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


_PORT = None


def _free_port_once():
    global _PORT
    if _PORT is None:
        _PORT = _free_port()
    return _PORT
