"""The optional neighbours of the layer (``vmoe_forward_ex``): router projection in front
(fused-moe/csrc/megakernel_v1.cu:455-489) and residual add behind, against plain references."""
import os

import numpy as np
import pytest
import torch

os.environ.setdefault("VMOE_NO_VLLM", "1")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,K,E", [(1, 1024, 8), (5, 4096, 512), (64, 4096, 512), (19, 2048, 100)])
def test_router_gemv_matches_f64(M, K, E, dtype):
    from sm120_moe_bench_b200 import ops
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, K, generator=g) * 0.05).to(dtype)
    got = ops.router_gemv(x.cuda(), w.cuda()).cpu()
    want = x.double() @ w.double().T
    # f32 accumulation of K products of magnitude ~0.05: absolute error far below 1e-4
    assert got.shape == (M, E)
    assert float((got.double() - want).abs().max()) <= 2e-5 * np.sqrt(K)
    # fixed summation order: bit-identical on repeat
    again = ops.router_gemv(x.cuda(), w.cuda()).cpu()
    assert torch.equal(got, again)


@pytest.mark.parametrize("path", [1, 2])
def test_gate_weight_in_equals_logits_in(path):
    """hidden + router matrix in: the layer routes on the logits of its own projection, and the result is the
    bits it produces when those same logits are handed in."""
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.CONFIG_TINY
    layer = synth.make_layer(cfg, seed=0)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]])
    if path == 2:
        routed.prepare()
    M = 6
    hidden, _ = synth.make_inputs(cfg, M, seed=3)
    g = torch.Generator().manual_seed(11)
    gate_w = (torch.randn(cfg.num_experts, cfg.hidden, generator=g) * 0.05).cuda()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=False, path=path))
    out_a = vm.fused_moe(hidden.cuda(), routed, ws, gate_weight=gate_w)
    ids_a = ws.view("topk_ids", torch.int32, M * cfg.topk).clone()
    logits = ops.router_gemv(hidden.cuda(), gate_w)
    out_b = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits)
    ids_b = ws.view("topk_ids", torch.int32, M * cfg.topk).clone()
    torch.cuda.synchronize()
    assert torch.equal(ids_a, ids_b)
    assert torch.equal(out_a, out_b)
    assert ws.status() == 0


@pytest.mark.parametrize("in_place", [False, True])
def test_residual_equals_separate_bf16_add(in_place):
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.CONFIG_TINY
    layer = synth.make_layer(cfg, seed=1)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    M = 9
    hidden, logits = synth.make_inputs(cfg, M, seed=4)
    hidden, logits = hidden.cuda(), logits.cuda()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=False, path=2))
    plain = vm.fused_moe(hidden, routed, ws, router_logits=logits)
    want = hidden + plain                                           # bf16 + bf16 -> f32 add, one rounding
    if in_place:
        x = hidden.clone()
        got = vm.fused_moe(x, routed, ws, router_logits=logits, residual=x, out=x)
        assert got.data_ptr() == x.data_ptr()
    else:
        got = vm.fused_moe(hidden, routed, ws, router_logits=logits, residual=hidden)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
