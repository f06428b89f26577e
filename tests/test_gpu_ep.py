"""Expert parallelism: the peer-memory dispatch / combine path against the single-GPU layer.

* world = 1 runs the whole chain (plan, dispatch into the rank's own slab, gather, permutation,
  tcgen05 experts with the epilogue storing into the combine slab, signal, combine) on one GPU;
* world = 2 runs as two child processes under torchrun when the box has at least two GPUs.
Outputs must be bit-identical to the single-GPU tensor-core path: same kernels per pair, fp32 rows,
same fixed-order sum."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_matches_fused_layer():
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ep, ops, synth
    cfg = synth.LayerConfig("ep1", 1024, 512, 16, 4, True)
    layer = synth.make_layer(cfg, seed=5)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare()
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, routed, shared, max_local_tokens=301)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 301, has_shared=True, path=2))
    try:
        # several calls: epochs advance, slabs are reused; 301 and 48 tokens take the token-major kernels (several units
        # per expert, unit sizes that are no multiple of four), the others the weights-as-rows kernel
        for M in (301, 48, 5, 0, 17):
            hidden, logits = synth.make_inputs(cfg, max(M, 1), seed=M)
            hidden, logits = hidden[:M].cuda().contiguous(), logits[:M].cuda().contiguous()
            out = moe.forward(hidden, logits)
            torch.cuda.synchronize()
            assert moe.status() == 0
            if M:
                ref = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared)
                assert torch.equal(out, ref)
    finally:
        moe.close()


def test_capacity_overflow_is_reported():
    from sm120_moe_bench_b200 import ep, ops, synth
    cfg = synth.LayerConfig("ep1", 1024, 512, 16, 4, False)
    layer = synth.make_layer(cfg, seed=5)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, routed, None, max_local_tokens=8, capacity=4)
    try:
        hidden, logits = synth.make_inputs(cfg, 8, seed=1)
        moe.forward(hidden.cuda(), logits.cuda())
        torch.cuda.synchronize()
        assert moe.status() == 8                      # VMOE_ERR_LIMIT
    finally:
        moe.close()


def test_unanswered_wait_times_out_and_the_device_stays_usable():
    """Failure detection without a fault: a world-2 context on ONE GPU whose second "rank" is a local buffer that
    nobody ever signals, wait limit 20 ms.  The gather and the combine give up, the status word reads
    VMOE_ERR_TIMEOUT, the output is not written, and a normal call afterwards succeeds.  (The reference's waits are
    unbounded: fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:156-167.)"""
    import ctypes as C
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ep, ops, synth
    from sm120_moe_bench_b200._lib import lib
    cfg = synth.LayerConfig("ep1", 1024, 512, 16, 4, True)
    layer = synth.make_layer(cfg, seed=5)
    half = ops.MoEWeights(*[t[:8].contiguous().cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare()
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, half, shared, max_local_tokens=8,
                               wait_limit_us=20_000, fake_world=2)
    try:
        hidden, logits = synth.make_inputs(cfg, 8, seed=1)
        out = torch.full((8, cfg.hidden), 7.0, dtype=torch.bfloat16, device="cuda")
        moe.forward(hidden.cuda(), logits.cuda(), out=out)
        torch.cuda.synchronize()
        assert moe.status() == 6                      # VMOE_ERR_TIMEOUT
        assert bool((out == 7.0).all())               # nothing was written
        assert moe.status() == 0                      # the read cleared the word
    finally:
        moe.close()
    # the context is intact: an ordinary call on the same device works
    full = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    ok = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, full, shared, max_local_tokens=8)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 8, has_shared=True, path=2))
    try:
        out = ok.forward(hidden.cuda(), logits.cuda())
        torch.cuda.synchronize()
        assert ok.status() == 0
        assert torch.equal(out, vm.fused_moe(hidden.cuda(), full, ws, router_logits=logits.cuda(), shared=shared))
    finally:
        ok.close()


def test_graph_replay_and_fused_residual_match_eager():
    """The exchange keeps its call number on the device, so the whole chain can be captured in a CUDA graph; a
    replay equals the eager call bit for bit, and the fused residual equals a separate bf16 add."""
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ep, ops, synth
    cfg = synth.LayerConfig("ep1", 1024, 512, 16, 4, True)
    layer = synth.make_layer(cfg, seed=5)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare()
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, routed, shared, max_local_tokens=24)
    try:
        hidden, logits = synth.make_inputs(cfg, 24, seed=9)
        hidden, logits = hidden.cuda(), logits.cuda()
        eager = moe.forward(hidden, logits).clone()
        with_res = moe.forward(hidden, logits, residual=hidden).clone()
        torch.cuda.synchronize()
        assert torch.equal(with_res, hidden + eager)
        out = torch.empty_like(hidden)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            moe.forward(hidden, logits, out=out)
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                moe.forward(hidden, logits, out=out)
        torch.cuda.synchronize()
        for _ in range(3):
            out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, eager)
        assert moe.status() == 0
        assert torch.equal(moe.forward(hidden, logits), eager)        # eager again after the replays
    finally:
        moe.close()


def test_hot_rank_rows_beyond_the_balanced_estimate():
    """The rows a rank receives do not follow from its own batch: here every token is routed to the same four
    experts, so they hold many more rows than the unit list of a balanced batch of this size would need.  The
    workspace is sized for the worst case and the result still equals the single-GPU layer."""
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ep, ops, synth
    cfg = synth.LayerConfig("ep1", 1024, 512, 16, 4, True)
    layer = synth.make_layer(cfg, seed=5)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare()
    M = 40
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, routed, shared, max_local_tokens=M)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2))
    try:
        hidden, logits = synth.make_inputs(cfg, M, seed=4)
        logits[:, [2, 5, 11, 13]] += 50.0
        out = moe.forward(hidden.cuda(), logits.cuda())
        torch.cuda.synchronize()
        assert moe.status() == 0
        assert torch.equal(out, vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits.cuda(), shared=shared))
    finally:
        moe.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_rank_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29610 + world),
           os.path.join(ROOT, "tests", "ep_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("EP_WORKER_OK") == world, res.stdout[-3000:]
