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


def test_rmsnorm_quantize_bit_exact():
    """vmoe_rmsnorm_quantize against oracle.moe.rmsnorm_quantize: normalised bf16 rows, FP4 codes and E4M3 scales
    bit for bit (hidden 4096: one block per thread; 7168: several; 512: idle threads)."""
    from oracle import moe as omoe
    from sm120_moe_bench_b200 import ops
    for K, rows in ((4096, 5), (7168, 3), (512, 9)):
        g = torch.Generator().manual_seed(K)
        x = (torch.randn(rows, K, generator=g) * 1.7).to(torch.bfloat16)
        x[0, :16] = 0
        gamma = (1.0 + 0.1 * torch.randn(K, generator=g)).float()
        got = ops.rmsnorm_quantize(x.cuda(), gamma.cuda(), 1e-6)
        torch.cuda.synchronize()
        y, packed, sf = omoe.rmsnorm_quantize(x.float().numpy(), gamma.numpy(), 1e-6)
        assert np.array_equal(got.normed.float().cpu().numpy(), y)
        assert np.array_equal(got.packed.cpu().numpy(), packed) and np.array_equal(got.sf.cpu().numpy(), sf)


@pytest.mark.parametrize("M", [3, 40, 300])
def test_fused_norm_behind_the_combine_and_quantised_input(M):
    """next_norm behind the combine equals the stand-alone kernel applied to the layer's output (+ residual), and a
    second layer fed those codes (hidden_quantized) equals the same layer fed the normalised bf16 rows: bit for bit.
    Batch 3 takes the one-CTA front, 40 the weights-as-rows kernel, 300 the token-major kernels."""
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.LayerConfig("mid", 512, 256, 12, 3, True)
    l1, l2 = synth.make_layer(cfg, seed=31), synth.make_layer(cfg, seed=32)
    dev = lambda six: ops.MoEWeights(*[t.cuda() for t in six]).prepare()
    r1, s1, r2, s2 = dev(l1["routed"]), dev(l1["shared"]), dev(l2["routed"]), dev(l2["shared"])
    hidden, logits = synth.make_inputs(cfg, M, seed=M)
    _, logits2 = synth.make_inputs(cfg, M, seed=M + 1)
    hidden, logits, logits2 = hidden.cuda(), logits.cuda(), logits2.cuda()
    gamma = (1.0 + 0.1 * torch.randn(cfg.hidden, generator=torch.Generator().manual_seed(1))).float().cuda()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2))
    plain = vm.fused_moe(hidden, r1, ws, router_logits=logits, shared=s1, residual=hidden).clone()
    rows = ops.QuantizedRows(M, cfg.hidden)
    fused = vm.fused_moe(hidden, r1, ws, router_logits=logits, shared=s1, residual=hidden, next_norm=(gamma, 1e-6), next_rows=rows).clone()
    alone = ops.rmsnorm_quantize(plain, gamma, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(fused, plain)
    assert torch.equal(rows.normed, alone.normed) and torch.equal(rows.packed, alone.packed) and torch.equal(rows.sf, alone.sf)
    a = vm.fused_moe(rows.normed, r2, ws, router_logits=logits2, shared=s2).clone()
    b = vm.fused_moe(None, r2, ws, router_logits=logits2, shared=s2, hidden_quantized=rows)
    torch.cuda.synchronize()
    assert ws.status() == 0 and torch.equal(a, b)
