"""Edge cases of the layer on the GPU: empty batch, every token on one expert, no local expert at all, zero
activation rows, zero / NaN block scales in the weights, the largest top-k.  Both kernel paths, against the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from tests import util

os.environ.setdefault("VMOE_NO_VLLM", "1")
pytestmark = pytest.mark.gpu

GEMV, TC = 1, 2
PATHS = [pytest.param(GEMV, id="gemv"), pytest.param(TC, id="tc")]


def _setup(cfg, seed, path, mutate=None):
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    layer = synth.make_layer(cfg, seed=seed)
    if mutate is not None:
        mutate(layer)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]])
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]) if cfg.shared else None
    if path == TC:
        routed.prepare()
        if shared is not None:
            shared.prepare()
    return vm, layer, routed, shared


def _oracle(layer, cfg, hidden, ids, w, expert_map=None):
    ow = util.to_oracle_weights(layer["routed"])
    osh = util.to_oracle_weights(layer["shared"]) if cfg.shared else None
    return omoe.moe_layer(hidden.float().numpy(), ids, w, ow, osh, expert_map=expert_map)


@pytest.mark.parametrize("path", PATHS)
def test_empty_batch(path):
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("mid", 512, 256, 12, 3, True)
    vm, layer, routed, shared = _setup(cfg, 1, path)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 8, has_shared=True, path=path))
    hidden = torch.empty(0, cfg.hidden, dtype=torch.bfloat16, device="cuda")
    logits = torch.empty(0, cfg.num_experts, dtype=torch.float32, device="cuda")
    out = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared)
    torch.cuda.synchronize()
    assert out.shape == (0, cfg.hidden) and ws.status() == 0


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M", [5, 70, 200, 600])
def test_every_token_on_the_same_experts(path, M):
    """All tokens pick experts 3 and 7 (in that order): two experts with M tokens each, the others empty.
    M = 70 / 200 / 600 takes the token-major kernels (128-token units) with several units per expert."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("skew", 512, 256, 12, 2, True)
    vm, layer, routed, shared = _setup(cfg, 2, path)
    hidden, _ = synth.make_inputs(cfg, M, seed=M)
    ids = np.tile(np.array([[3, 7]], np.int32), (M, 1))
    g = np.random.default_rng(M)
    w = g.uniform(0.1, 0.9, size=(M, 2)).astype(np.float32)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=path))
    out = vm.fused_moe(hidden.cuda(), routed, ws, topk_ids=torch.from_numpy(ids).cuda(),
                       topk_weights=torch.from_numpy(w).cuda(), shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    offs = ws.view("expert_offsets", torch.int32, cfg.num_experts + 2).cpu().numpy()
    counts = np.diff(offs[:cfg.num_experts + 1])
    assert counts[3] == M and counts[7] == M and counts.sum() == 2 * M
    util.assert_output_close(out.float().cpu().numpy(), _oracle(layer, cfg, hidden, ids, w))


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("with_shared", [False, True])
def test_no_local_expert(path, with_shared):
    """An expert_map of all -1 (this rank owns none of the chosen experts): the routed part is zero, the shared
    expert (when present) is the whole output."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("nolocal", 512, 256, 12, 3, with_shared)
    vm, layer, routed, shared = _setup(cfg, 3, path)
    M = 6
    hidden, logits = synth.make_inputs(cfg, M, seed=9)
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    emap = np.full(cfg.num_experts, -1, np.int32)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=with_shared, path=path))
    out = vm.fused_moe(hidden.cuda(), routed, ws, topk_ids=torch.from_numpy(ids).cuda(), topk_weights=torch.from_numpy(w).cuda(),
                       shared=shared, expert_map=torch.from_numpy(emap).cuda())
    torch.cuda.synchronize()
    assert ws.status() == 0
    got = out.float().cpu().numpy()
    if not with_shared:
        assert np.array_equal(got, np.zeros_like(got))
    else:
        util.assert_output_close(got, _oracle(layer, cfg, hidden, ids, w, expert_map=emap))


@pytest.mark.parametrize("path", PATHS)
def test_zero_rows_and_degenerate_weight_scales(path):
    """Token rows of zeros (block amax 0: scale floored, codes 0), weight blocks whose scale byte is 0, and NaN
    scale bytes (0x7F), which decode to zero (fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:48-55)."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("degen", 512, 256, 12, 3, True)

    def mutate(layer):
        w13, w13_sf, _, w2, w2_sf, _ = layer["routed"]
        w13_sf[:, ::5, 1] = 0                       # zero scales
        w13_sf[:, 1::7, 2] = 0x7F                   # NaN scales
        w2_sf[:, ::3, 0] = 0x7F
        w2_sf[:, 2::9, 3] = 0

    vm, layer, routed, shared = _setup(cfg, 4, path, mutate)
    M = 10
    hidden, logits = synth.make_inputs(cfg, M, seed=12)
    hidden[2] = 0
    hidden[7, :256] = 0
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=path))
    out = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits.cuda(), shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.array_equal(got[2], np.zeros_like(got[2]))          # a zero token stays zero through SiLU * up
    util.assert_output_close(got, _oracle(layer, cfg, hidden, ids, w))


@pytest.mark.parametrize("path", PATHS)
def test_largest_topk(path):
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("t16", 512, 256, 40, 16, False)
    vm, layer, routed, shared = _setup(cfg, 5, path)
    M = 7
    hidden, logits = synth.make_inputs(cfg, M, seed=13)
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=False, path=path))
    out = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits.cuda())
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert np.array_equal(ws.view("topk_ids", torch.int32, M * 16).cpu().numpy().reshape(M, 16), ids)
    util.assert_output_close(out.float().cpu().numpy(), _oracle(layer, cfg, hidden, ids, w))
