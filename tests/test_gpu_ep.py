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
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, routed, shared, max_local_tokens=48)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 48, has_shared=True, path=2))
    try:
        for M in (48, 5, 0, 17):                       # several calls: epochs advance, slabs are reused
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


@pytest.mark.parametrize("world", [2, 4])
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
