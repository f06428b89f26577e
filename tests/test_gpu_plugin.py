"""The operator classes (the drop-in boundary) on the GPU: ``VerdictMoEExperts.apply`` with the
reference's exact call signature (fused-moe/verdict_moe.py:421-438) and ``VerdictMoEMonolithic.apply``
(router logits in), against the C-ABI layer and the oracle.  Cases follow the reference's own
mocked-backend test (fused-moe/test_cuda_graph_safety.py:325-386): M = 2, an expert_map with -1
entries, router weight applied on the input, repeat-call determinism, no allocation between calls."""
import os

import numpy as np
import pytest
import torch

os.environ.setdefault("VMOE_NO_VLLM", "1")
pytestmark = pytest.mark.gpu


class _Quant:
    """The quant-config attributes the class reads (fused-moe/verdict_moe.py:499-503, :519-520)."""
    def __init__(self, routed, convention):
        a13 = torch.full_like(routed.w13_gs, 0.37)        # a made-up static activation scale
        a2 = torch.full_like(routed.w2_gs, 1.9)
        if convention == "product":                        # framework pre-multiplies: g = a * w_scale_2, a_gscale = 1 / a
            self.g1_alphas, self.a1_gscale = routed.w13_gs * a13, 1.0 / a13
            self.g2_alphas, self.a2_gscale = routed.w2_gs * a2, 1.0 / a2
        else:                                              # framework hands the raw weight global scale
            self.g1_alphas, self.a1_gscale = routed.w13_gs.clone(), 1.0 / a13
            self.g2_alphas, self.a2_gscale = routed.w2_gs.clone(), 1.0 / a2
        self.w1_scale = routed.w13_sf.view(torch.float8_e4m3fn)
        self.w2_scale = routed.w2_sf.view(torch.float8_e4m3fn)


class _MoeCfg:
    experts_per_token = 2


@pytest.fixture(scope="module")
def setup():
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.CONFIG_TINY
    layer = synth.make_layer(cfg, seed=0)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]])
    return vm, cfg, layer, routed


@pytest.mark.parametrize("convention", ["product", "weight"])
@pytest.mark.parametrize("kernel_path", [1, 2])
def test_apply_reference_signature(setup, convention, kernel_path):
    vm, cfg, layer, routed = setup
    from oracle import moe as omoe
    from sm120_moe_bench_b200 import synth
    from sm120_moe_bench_b200.verdict_moe import VerdictMoEExperts
    from tests import util
    M = 2
    hidden, logits = synth.make_inputs(cfg, M, seed=11)
    ids_ref, w_ref = omoe.route(logits.numpy(), cfg.topk)
    op = VerdictMoEExperts(_MoeCfg(), _Quant(routed, convention))
    op.alpha_convention = convention
    op.kernel_path = kernel_path
    out = torch.full((M, cfg.hidden), 7.0, dtype=torch.bfloat16, device="cuda")
    # framework hands int64 ids and bf16-adjacent dtypes: the class converts, as the reference's copy_() does
    args = (out, hidden.cuda(), routed.w13, routed.w2, torch.from_numpy(w_ref).cuda(),
            torch.from_numpy(ids_ref).cuda().long(), "SILU", cfg.num_experts, None, None, None, None, None, None, False)
    op.apply(*args)
    torch.cuda.synchronize()
    ow = omoe.ExpertWeights(*[t.numpy() for t in layer["routed"]])
    ref = omoe.moe_layer(hidden.float().numpy(), ids_ref, w_ref, ow)
    util.assert_output_close(out.float().cpu().numpy(), ref)
    # repeat call: bit-identical output, no device allocation (CUDA-graph safety of the reference class)
    first = out.clone()
    before = torch.cuda.memory_allocated()
    op.apply(*args)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.equal(out, first)


def test_both_alpha_conventions_agree(setup):
    vm, cfg, layer, routed = setup
    from sm120_moe_bench_b200 import synth
    from sm120_moe_bench_b200.verdict_moe import VerdictMoEExperts
    hidden, logits = synth.make_inputs(cfg, 4, seed=3)
    ids, w = vm.route(logits.cuda(), cfg.topk)
    outs = []
    for conv in ("product", "weight"):
        op = VerdictMoEExperts(_MoeCfg(), _Quant(routed, conv))
        op.alpha_convention = conv
        out = torch.empty(4, cfg.hidden, dtype=torch.bfloat16, device="cuda")
        op.apply(out, hidden.cuda(), routed.w13, routed.w2, w, ids, "SILU", cfg.num_experts, None, None, None,
                 None, None, None, False)
        outs.append(out)
    torch.cuda.synchronize()
    # a * w * (1 / a) differs from w by one or two float32 roundings of the per-expert scalar
    np.testing.assert_allclose(outs[0].float().cpu().numpy(), outs[1].float().cpu().numpy(), rtol=2e-2, atol=1e-6)


def test_expert_map_and_router_weight_on_input(setup):
    vm, cfg, layer, routed = setup
    from sm120_moe_bench_b200 import ops, synth
    from sm120_moe_bench_b200.verdict_moe import VerdictMoEExperts
    hidden, logits = synth.make_inputs(cfg, 6, seed=5)
    ids, w = vm.route(logits.cuda(), cfg.topk)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 6))
    full = vm.fused_moe(hidden.cuda(), routed, ws, topk_ids=ids, topk_weights=w).float()
    # expert parallel: this "rank" holds experts 2..5 only (fused-moe/test_cuda_graph_safety.py: expert_map=[0,1,-1])
    emap = torch.full((cfg.num_experts,), -1, dtype=torch.int64)
    emap[2:6] = torch.arange(4)
    part = ops.MoEWeights(*[t[2:6].contiguous().cuda() for t in layer["routed"]])
    rest_map = torch.full((cfg.num_experts,), -1, dtype=torch.int64)
    rest_map[[0, 1, 6, 7]] = torch.arange(4)
    rest = ops.MoEWeights(*[t[[0, 1, 6, 7]].contiguous().cuda() for t in layer["routed"]])
    total = torch.zeros_like(full)
    for wts, m in ((part, emap), (rest, rest_map)):
        op = VerdictMoEExperts(_MoeCfg(), _Quant(wts, "product"))
        out = torch.empty(6, cfg.hidden, dtype=torch.bfloat16, device="cuda")
        op.apply(out, hidden.cuda(), wts.w13, wts.w2, w, ids, "SILU", cfg.num_experts, m.cuda(), None, None, None,
                 None, None, False)
        total += out.float()
    torch.cuda.synchronize()
    assert (total - full).abs().max().item() <= 2 ** -6 * full.abs().max().item()
    # router weight applied on the input (top-1 routing in the frameworks that use it)
    ids1, w1 = ids[:, :1].contiguous(), w[:, :1].contiguous()
    op = VerdictMoEExperts(_MoeCfg(), _Quant(routed, "product"))
    out = torch.empty(6, cfg.hidden, dtype=torch.bfloat16, device="cuda")
    op.apply(out, hidden.cuda(), routed.w13, routed.w2, w1, ids1, "SILU", cfg.num_experts, None, None, None, None,
             None, None, True)
    ws1 = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, 1, 6))
    scaled = (hidden.cuda() * w1.to(torch.bfloat16)).contiguous()
    ref = vm.fused_moe(scaled, routed, ws1, topk_ids=ids1, topk_weights=torch.ones_like(w1))
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_monolithic_router_logits_in(setup):
    vm, cfg, layer, routed = setup
    from sm120_moe_bench_b200 import synth
    from sm120_moe_bench_b200.verdict_moe import VerdictMoEMonolithic
    hidden, logits = synth.make_inputs(cfg, 5, seed=9)
    op = VerdictMoEMonolithic(_MoeCfg(), _Quant(routed, "product"))
    out = op.apply(hidden.cuda(), routed.w13, routed.w2, logits.cuda(), "SILU", cfg.num_experts, None, None, False)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 5))
    ref = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits.cuda())
    torch.cuda.synchronize()
    # alpha = (a * w) * (1 / a): within float32 rounding of the direct scale
    np.testing.assert_allclose(out.float().cpu().numpy(), ref.float().cpu().numpy(), rtol=2e-2, atol=1e-6)
    with pytest.raises(ValueError):
        op.apply(hidden.cuda(), routed.w13, routed.w2, logits.cuda(), "SILU", cfg.num_experts, None, None, False,
                 num_expert_group=4)


def test_apply_inside_cuda_graph_after_weight_hook(setup):
    """What a serving engine does with the class: ``process_weights_after_loading`` once (binds the weights and
    builds the scale atoms), one warm-up call (sizes the workspace), then ``apply`` captured in a CUDA graph and
    replayed with new inputs in the same buffers.  Replays equal eager calls bit for bit and allocate nothing
    (the buffer pre-allocation property of fused-moe/test_cuda_graph_safety.py:325-386)."""
    vm, cfg, layer, routed = setup
    import types

    from oracle import moe as omoe
    from sm120_moe_bench_b200 import synth
    from sm120_moe_bench_b200.verdict_moe import VerdictMoEExperts
    M = 4
    op = VerdictMoEExperts(_MoeCfg(), _Quant(routed, "weight"))
    op.alpha_convention = "weight"
    op.kernel_path = 2
    op.process_weights_after_loading(types.SimpleNamespace(w13_weight=routed.w13, w2_weight=routed.w2))
    assert op._weights is not None and op._weights.w13_sf_atoms is not None
    hidden = torch.zeros(M, cfg.hidden, dtype=torch.bfloat16, device="cuda")
    wts = torch.zeros(M, cfg.topk, dtype=torch.float32, device="cuda")
    ids = torch.zeros(M, cfg.topk, dtype=torch.int32, device="cuda")
    out = torch.zeros(M, cfg.hidden, dtype=torch.bfloat16, device="cuda")
    args = (out, hidden, routed.w13, routed.w2, wts, ids, "SILU", cfg.num_experts, None, None, None, None, None, None, False)

    def load(seed):
        h, logits = synth.make_inputs(cfg, M, seed=seed)
        i, w = omoe.route(logits.numpy(), cfg.topk)
        hidden.copy_(h.cuda()); ids.copy_(torch.from_numpy(i).cuda()); wts.copy_(torch.from_numpy(w).cuda())

    load(1)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        op.apply(*args)                                   # warm-up on the capture stream: workspace, tensor maps
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        op.apply(*args)
    for seed in (2, 3):
        load(seed)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        replayed = out.clone()
        op.apply(*args)
        torch.cuda.synchronize()
        assert torch.equal(out, replayed)
