"""Host-side logic of the expert-parallel path on CPU: the partition helpers, and a world-size-2
gloo run of the handle exchange pattern and of the oracle's expert-parallel decomposition."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_partition_helpers():
    from sm120_moe_bench_b200 import ep
    assert ep.expert_partition(512, 8, 3) == (192, 64)
    m = ep.expert_map_for_rank(512, 8, 3)
    assert m.dtype == torch.int32 and m[191] == -1 and m[192] == 0 and m[255] == 63 and m[256] == -1
    assert int((m >= 0).sum()) == 64
    with pytest.raises(ValueError):
        ep.expert_partition(10, 4, 0)
    assert ep.default_capacity(192, 10, 8) == 192 * 11


def _gloo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import moe as omoe
    from sm120_moe_bench_b200 import ep, synth
    # (1) the 64-byte handle exchange used at construction: rank-ordered all_gather_object
    handle = bytes([rank]) * 64
    got = [None] * world
    dist.all_gather_object(got, handle)
    assert [g[0] for g in got] == list(range(world)) and all(len(g) == 64 for g in got)
    # (2) every rank computes its experts' share for ALL tokens (gathered), owners sum the shares
    cfg = synth.LayerConfig("cpu-ep", 256, 128, 8, 2, False)
    layer = synth.make_layer(cfg, seed=1)
    hidden, logits = synth.make_inputs(cfg, 6, seed=rank)          # each rank's own tokens
    hs = [None] * world; ls = [None] * world
    dist.all_gather_object(hs, hidden.float().numpy()); dist.all_gather_object(ls, logits.numpy())
    first, per = ep.expert_partition(cfg.num_experts, world, rank)
    emap = ep.expert_map_for_rank(cfg.num_experts, world, rank).numpy()
    mine = omoe.ExpertWeights(*[t[first:first + per].numpy() for t in layer["routed"]])
    shares = []
    for src in range(world):
        ids, w = omoe.route(ls[src], cfg.topk)
        _, st = omoe.moe_layer(hs[src], ids, w, mine, expert_map=emap, return_stages=True)
        shares.append(st["pair_out"])                               # [M, T, K] rows of this rank's experts
    allshares = [None] * world
    dist.all_gather_object(allshares, shares)
    ids, w = omoe.route(ls[rank], cfg.topk)
    acc = np.zeros_like(hs[rank])
    for j in range(cfg.topk):                                        # fixed order over pairs
        rows = sum(allshares[r][rank][:, j] for r in range(world))  # exactly one rank contributes a non-zero row
        acc = (acc + rows).astype(np.float32)
    from oracle import nvfp4
    full = omoe.ExpertWeights(*[t.numpy() for t in layer["routed"]])
    ref = omoe.moe_layer(hs[rank], ids, w, full)
    assert np.array_equal(nvfp4.bf16_round(acc), ref)
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, "ok"))


def test_two_rank_gloo_exchange_and_decomposition():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert sorted(q.get(timeout=5) for _ in range(2)) == [(0, "ok"), (1, "ok")]
