"""GPU parity of the fused layer through the C ABI against the CPU oracle, with stage-wise checks
that separate exact integer work from the floating-point tolerance."""
import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import nvfp4
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vm():
    import sm120_moe_bench_b200 as pkg
    return pkg


GEMV, TC = 1, 2      # vmoe_path values: streaming GEMV on CUDA cores / tcgen05 tensor cores
PATHS = [pytest.param(GEMV, id="gemv"), pytest.param(TC, id="tc")]


def _device_layer(vm, layer, prepare=True):
    from sm120_moe_bench_b200 import ops
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]])
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]) if layer["shared"] is not None else None
    if prepare:
        routed.prepare()
        if shared is not None:
            shared.prepare()
    return routed, shared


def _run_and_check(vm, cfg, layer, hidden, logits, M, expert_subset=True, use_logits=True, path=GEMV):
    from sm120_moe_bench_b200 import ops
    routed, shared = _device_layer(vm, layer)
    shape = vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=cfg.shared, path=path)
    ws = vm.Workspace(shape)
    hid_d, log_d = hidden.cuda(), logits.cuda()
    ids_ref, w_ref = omoe.route(logits.cpu().numpy(), cfg.topk)
    if use_logits:
        out = vm.fused_moe(hid_d, routed, ws, router_logits=log_d, shared=shared)
    else:
        out = vm.fused_moe(hid_d, routed, ws, topk_ids=torch.from_numpy(ids_ref).cuda(),
                           topk_weights=torch.from_numpy(w_ref).cuda(), shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    S = M * cfg.topk + (M if cfg.shared else 0)
    if use_logits:
        ids_dev = ws.view("topk_ids", torch.int32, M * cfg.topk).cpu().numpy().reshape(M, cfg.topk)
        assert np.array_equal(ids_dev, ids_ref)
        w_dev = ws.view("topk_weights", torch.float32, M * cfg.topk).cpu().numpy().reshape(M, cfg.topk)
    else:
        w_dev = w_ref
    # ---- oracle on the same bytes (device router weights: isolates the layer from expf last bits)
    used = np.unique(ids_ref)
    ow = util.to_oracle_weights(layer["routed"], used if expert_subset else None)
    osh = util.to_oracle_weights(layer["shared"]) if cfg.shared else None
    ref, st = omoe.moe_layer(hidden.float().cpu().numpy(), ids_ref, w_dev, ow, osh, return_stages=True)
    # ---- a6: activation codes and scales bit-exact
    act_q = ws.view("act_q", torch.uint8, M * cfg.hidden // 2).cpu().numpy().reshape(M, -1)
    act_sf = ws.view("act_sf", torch.uint8, M * cfg.hidden // 16).cpu().numpy().reshape(M, -1)
    assert np.array_equal(act_q, st["xq"]) and np.array_equal(act_sf, st["xsf"])
    # ---- a9: intermediate FP4 codes per sorted slot: equal up to rare rounding flips
    t = ws.tables(M)
    inter_q = ws.view("inter_q", torch.uint8, S * cfg.inter // 2).cpu().numpy().reshape(S, -1)
    inter_sf = ws.view("inter_sf", torch.uint8, S * cfg.inter // 16).cpu().numpy().reshape(S, -1)
    sp = t["sorted_pair"].numpy()
    flips = 0; sf_flips = 0
    oracle_inter_q = np.zeros_like(inter_q); oracle_inter_sf = np.zeros_like(inter_sf)
    for slot, p in enumerate(sp):
        key = (int(p) // cfg.topk, int(p) % cfg.topk) if p < M * cfg.topk else (int(p) - M * cfg.topk, cfg.topk)
        q, sf, _ = st["inter"][key]
        oracle_inter_q[slot], oracle_inter_sf[slot] = q, sf
    flips = np.mean(nvfp4.unpack_nibbles(inter_q) != nvfp4.unpack_nibbles(oracle_inter_q))
    sf_flips = np.mean(inter_sf != oracle_inter_sf)
    assert flips <= util.INTER_FLIP_RATE_MAX and sf_flips <= util.INTER_FLIP_RATE_MAX, (flips, sf_flips)
    # ---- a10: down projection fed the DEVICE's own intermediate -> tight tolerance
    pair_out = ws.view("pair_out", torch.float32, S * cfg.hidden).cpu().numpy().reshape(S, cfg.hidden)
    sw = t["scatter_weights"].numpy()
    worst = 0.0
    rng = np.random.default_rng(0)
    for slot in rng.choice(S, size=min(S, 24), replace=False):
        p = int(sp[slot])
        if p < M * cfg.topk:
            e = int(ids_ref.reshape(-1)[p]); W = ow; a2 = W.w2_gs[e]
        else:
            e = 0; W = osh; a2 = W.w2_gs[0]
        sq = nvfp4.dequantize(inter_q[slot], inter_sf[slot])
        w2 = nvfp4.dequantize(W.w2[e], W.w2_sf[e])
        y = (w2.astype(np.float64) @ sq.astype(np.float64)) * np.float64(np.float32(sw[slot] * a2))
        worst = max(worst, util.rel_l2(pair_out[slot], y.astype(np.float32)))
    assert worst <= 1e-5, worst
    # ---- a11: combine is the fixed-order fp32 sum of the device's own rows, bit-exact
    acc = np.zeros((M, cfg.hidden), np.float32)
    ps = t["pair_slot"].numpy().reshape(M, cfg.topk)
    for j in range(cfg.topk):
        acc = (acc + pair_out[ps[:, j]]).astype(np.float32)
    if cfg.shared:
        base = int(t["expert_offsets"][cfg.num_experts])
        acc = (acc + pair_out[base:base + M]).astype(np.float32)
    got = out.float().cpu().numpy()
    assert np.array_equal(got, nvfp4.bf16_round(acc))
    # ---- whole layer vs oracle
    return util.assert_output_close(got, ref), float(flips)


@pytest.mark.parametrize("path", PATHS)
def test_config_tiny(vm, path):
    """BASELINE config 1: hidden 1024, 8 experts, top-2, intermediate 512, 4 tokens, seed 0."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_TINY
    layer = synth.make_layer(cfg, seed=0)
    hidden, logits = synth.make_inputs(cfg, 4, seed=0)
    _run_and_check(vm, cfg, layer, hidden, logits, 4, expert_subset=False, use_logits=True, path=path)
    _run_and_check(vm, cfg, layer, hidden, logits, 4, expert_subset=False, use_logits=False, path=path)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M", [1, 3, 16, 50, 150, 300])
def test_small_shapes_with_shared(vm, M, path):
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("mid", 512, 256, 12, 3, True)
    layer = synth.make_layer(cfg, seed=3)
    hidden, logits = synth.make_inputs(cfg, M, seed=M)
    _run_and_check(vm, cfg, layer, hidden, logits, M, expert_subset=False, path=path)


@pytest.mark.parametrize("hidden,inter,E,T,shared,M", [
    (768, 768, 5, 1, True, 9),        # odd k-block counts: one k-block per stage in the down items
    (768, 256, 5, 5, False, 2),       # every expert on every token, no shared expert
    (1024, 768, 20, 16, True, 3),     # the largest top-k
    (512, 512, 33, 4, True, 33),      # expert and token counts that are not multiples of anything
    (2048, 256, 7, 2, False, 100),    # token-major kernels, no shared expert
    (768, 768, 6, 3, True, 130),      # token-major kernels with an odd k-block count
])
def test_assorted_shapes_on_the_tensor_core_path(vm, hidden, inter, E, T, shared, M):
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("odd", hidden, inter, E, T, shared)
    layer = synth.make_layer(cfg, seed=hidden + E)
    hid, logits = synth.make_inputs(cfg, M, seed=M + T)
    _run_and_check(vm, cfg, layer, hid, logits, M, expert_subset=False, path=TC)


def test_prepared_scale_layout(vm):
    """vmoe_prepare_sf: linear [rows, K/16] -> [rows/128][K/64][32][4][4] atoms, NaN bytes -> 0."""
    from sm120_moe_bench_b200._lib import lib
    g = torch.Generator().manual_seed(11)
    rows, K = 256, 512
    sf = torch.randint(0, 0x7F, (rows, K // 16), dtype=torch.uint8, generator=g)
    sf[3, 5] = 0x7F
    atoms = torch.full((rows * K // 16,), 0xEE, dtype=torch.uint8, device="cuda")
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.vmoe_prepare_sf(sf.cuda().data_ptr(), rows, K, atoms.data_ptr(), bad.data_ptr(), None) == 0
    torch.cuda.synchronize()
    ref = sf.clone(); ref[3, 5] = 0
    # [rows/128][r/32 (4)][r%32 (32)][K/64][kb%4] -> [rows/128][K/64][r%32][r/32][kb%4]
    ref = ref.view(rows // 128, 4, 32, K // 64, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)
    assert torch.equal(atoms.cpu(), ref) and int(bad.item()) == 0
    sf[0, 0] = 0x85
    assert lib.vmoe_prepare_sf(sf.cuda().data_ptr(), rows, K, atoms.data_ptr(), bad.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 1


@pytest.fixture(scope="module")
def large_layer():
    from sm120_moe_bench_b200 import synth
    return synth.make_layer(synth.CONFIG_LARGE, seed=0, device="cuda")


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M", [1, 4])
def test_config_large_decode(vm, large_layer, M, path):
    """BASELINE config 2 (hidden 4096, 512 experts top-10 + shared, intermediate 1024) at the batch
    sizes the oracle finishes in seconds; only the experts the batch touches are copied back."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_LARGE
    hidden, logits = synth.make_inputs(cfg, M, seed=M)
    _run_and_check(vm, cfg, large_layer, hidden, logits, M, expert_subset=True, path=path)


@pytest.mark.parametrize("path", PATHS)
def test_config_large_bs64_properties(vm, large_layer, path):
    """Batch 64 at full size, checked through size-independent properties: (1) a token's output does
    not depend on which other tokens share the batch (rows of the bs-64 run equal bs-1 runs bit for
    bit, as each token only uses its own top-k: fused-moe/test_expert_union.py:228-405), (2) run-twice
    determinism (fused-moe/test_cuda_graph_safety.py:366-386)."""
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.CONFIG_LARGE
    routed, shared = _device_layer(vm, large_layer)
    hidden, logits = synth.make_inputs(cfg, 64, seed=64)
    hid_d, log_d = hidden.cuda(), logits.cuda()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 64, has_shared=True, path=path))
    out1 = vm.fused_moe(hid_d, routed, ws, router_logits=log_d, shared=shared).clone()
    out2 = vm.fused_moe(hid_d, routed, ws, router_logits=log_d, shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert torch.equal(out1, out2)
    for m in (0, 17, 63):
        o = vm.fused_moe(hid_d[m:m + 1].contiguous(), routed, ws, router_logits=log_d[m:m + 1].contiguous(), shared=shared)
        assert torch.equal(o[0], out1[m])
    assert torch.isfinite(out1.float()).all() and out1.float().abs().max() > 0


def test_config_large_prefill_properties(vm, large_layer):
    """BASELINE config 3 at full size (8192 tokens, token-major tcgen05 tiles), through size-independent
    properties: run-twice determinism, and single rows against batch-1 runs of the same tokens (different
    kernels, so within the layer tolerance rather than bit for bit), uniform and Zipf-skewed routing."""
    from sm120_moe_bench_b200 import synth
    from tests import util
    cfg = synth.CONFIG_LARGE
    routed, shared = _device_layer(vm, large_layer)
    M = 8192
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=TC))
    ws1 = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 1, has_shared=True, path=TC))
    for zipf in (None, 1.2):
        hidden, logits = synth.make_inputs(cfg, M, seed=3, device="cuda", zipf_s=zipf)
        out1 = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared).clone()
        out2 = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared)
        torch.cuda.synchronize()
        assert ws.status() == 0
        assert torch.equal(out1, out2)
        assert torch.isfinite(out1.float()).all()
        t = ws.tables(M)
        assert t["num_slots"] == M * (cfg.topk + 1)
        for m in (0, 4097, 8191):
            o = vm.fused_moe(hidden[m:m + 1].contiguous(), routed, ws1, router_logits=logits[m:m + 1].contiguous(), shared=shared)
            util.assert_output_close(out1[m].float().cpu().numpy(), o[0].float().cpu().numpy())


def _oracle_rows(cfg, layer, hidden, ids_dev, w_dev, rows):
    """The oracle on a few token rows of a large batch.  A token's output only depends on its own top-k experts
    (and the shared one), so only those are copied back and dequantised: the cost of a batch-1 oracle run per row."""
    ids = ids_dev[rows].cpu().numpy()
    w = w_dev[rows].cpu().numpy()
    ow = util.to_oracle_weights(layer["routed"], np.unique(ids))
    osh = util.to_oracle_weights(layer["shared"]) if cfg.shared else None
    return omoe.moe_layer(hidden[rows].float().cpu().numpy(), ids, w, ow, osh)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M", [16, 64])
def test_config_large_decode_oracle_rows(vm, large_layer, M, path):
    """BASELINE config 2 at batch 16 and 64: three token rows of the batch against the oracle (router ids bit for
    bit for the whole batch, output within the layer tolerance)."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_LARGE
    routed, shared = _device_layer(vm, large_layer)
    hidden, logits = synth.make_inputs(cfg, M, seed=M)
    hid_d, log_d = hidden.cuda(), logits.cuda()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=path))
    out = vm.fused_moe(hid_d, routed, ws, router_logits=log_d, shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    ids_dev = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
    w_dev = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
    ids_ref, _ = omoe.route(logits.numpy(), cfg.topk)
    assert np.array_equal(ids_dev.cpu().numpy(), ids_ref)
    rows = [0, M // 2 + 1, M - 1]
    ref = _oracle_rows(cfg, large_layer, hid_d, ids_dev, w_dev, rows)
    util.assert_output_close(out[rows].float().cpu().numpy(), ref)


@pytest.mark.parametrize("zipf", [None, 1.2])
def test_config_large_prefill_oracle_rows(vm, large_layer, zipf):
    """BASELINE config 3 (8192 tokens, token-major tcgen05 kernels), uniform and Zipf(1.2) routing: three token
    rows against the oracle, router ids of 256 sampled rows bit for bit."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_LARGE
    routed, shared = _device_layer(vm, large_layer)
    M = 8192
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=TC))
    hidden, logits = synth.make_inputs(cfg, M, seed=3, device="cuda", zipf_s=zipf)
    out = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    ids_dev = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
    w_dev = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
    sample = torch.arange(0, M, 32)
    lg = logits[sample.cuda()].cpu().numpy()
    ids_ref, _ = omoe.route(lg, cfg.topk)
    ok = np.array([omoe.route_ids_are_unambiguous(lg[i:i + 1], cfg.topk) for i in range(len(lg))])
    assert ok.mean() > 0.99
    assert np.array_equal(ids_dev[sample.cuda()].cpu().numpy()[ok], ids_ref[ok])
    rows = [0, 4097, 8191]
    ref = _oracle_rows(cfg, large_layer, hidden, ids_dev, w_dev, rows)
    util.assert_output_close(out[rows].float().cpu().numpy(), ref)


@pytest.mark.parametrize("case", [
    pytest.param((512, 256, 8, 2, 1024, None), id="8experts-1024"),       # two or three units per expert
    pytest.param((512, 256, 8, 2, 1500, None), id="8experts-1500"),       # odd unit counts: half-empty pairs
    pytest.param((1024, 512, 16, 4, 2048, 1.2), id="16experts-zipf"),     # hot experts with many pairs, cold ones with one unit
])
def test_cta_pair_kernels_match_single_cta_kernels(vm, monkeypatch, case):
    """The token-major projections on CTA pairs (tcgen05 cta_group::2, opted into with VMOE_PF_PAIR) against the
    single-CTA kernels on the same inputs: the same products accumulated in the same order, so bit for bit; three
    rows of the pair run against the oracle as well."""
    from sm120_moe_bench_b200 import synth
    K, N, E, T, M, zipf = case
    cfg = synth.LayerConfig("pair", K, N, E, T, True)
    layer = synth.make_layer(cfg, seed=5, device="cuda")
    routed, shared = _device_layer(vm, layer)
    ws = vm.Workspace(vm.MoEShape(K, N, E, T, M, has_shared=True, path=TC))
    hidden, logits = synth.make_inputs(cfg, M, seed=9, device="cuda", zipf_s=zipf)
    outs = {}
    for pair in ("0", "3"):                                  # bit 0: gate_up on pairs, bit 1: down on pairs
        monkeypatch.setenv("VMOE_PF_PAIR", pair)
        outs[pair] = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared).clone()
        torch.cuda.synchronize()
        assert ws.status() == 0
    assert torch.equal(outs["0"], outs["3"])
    ids_dev = ws.view("topk_ids", torch.int32, M * T).view(M, T).clone()
    w_dev = ws.view("topk_weights", torch.float32, M * T).view(M, T).clone()
    rows = [0, M // 2 + 1, M - 1]
    ref = _oracle_rows(cfg, layer, hidden, ids_dev, w_dev, rows)
    util.assert_output_close(outs["3"][rows].float().cpu().numpy(), ref)


def test_bf16_pair_rows_option_stays_within_its_stated_error(vm, monkeypatch):
    """VMOE_PAIR_ROWS_BF16=1 (large batches): the down projection leaves its per-pair rows as bf16, the combine still
    sums them in fp32 in the fixed order.  A second rounding per pair: not bit-exact, measured at 2.7e-3 relative L2 on
    the 8192-token layer; here the bound the option is documented with (5e-3, cosine >= 0.9999) against the oracle, and
    the default path on the same inputs within the ordinary tolerance."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("rows16", 1024, 512, 16, 4, True)
    M = 2048
    layer = synth.make_layer(cfg, seed=11, device="cuda")
    routed, shared = _device_layer(vm, layer)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=TC))
    hidden, logits = synth.make_inputs(cfg, M, seed=12, device="cuda")
    outs = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("VMOE_PAIR_ROWS_BF16", flag)
        outs[flag] = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared).clone()
        torch.cuda.synchronize()
        assert ws.status() == 0
    ids_dev = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
    w_dev = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
    rows = [0, 5, M // 2 + 1, M - 1]
    ref = _oracle_rows(cfg, layer, hidden, ids_dev, w_dev, rows)
    util.assert_output_close(outs["0"][rows].float().cpu().numpy(), ref)
    got = outs["1"][rows].float().cpu().numpy()
    assert util.cosine(got, ref) >= 0.9999 and util.rel_l2(got, ref) <= 5e-3
    assert not torch.equal(outs["0"], outs["1"])          # the option really took the other path


def test_wide_shape_on_the_tensor_core_path(vm):
    """Hidden 7168, intermediate 2048 (beyond what the streaming GEMV kernels take): the tensor-core path has no
    such cap.  Four experts, top-2 + shared; decode (weights-as-rows kernel) and a 160-token batch (token-major)."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("wide", 7168, 2048, 4, 2, True)
    layer = synth.make_layer(cfg, seed=21, device="cuda")
    routed, shared = _device_layer(vm, layer)
    for M in (5, 160):
        hidden, logits = synth.make_inputs(cfg, M, seed=M, device="cuda")
        ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=TC))
        out = vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared)
        torch.cuda.synchronize()
        assert ws.status() == 0
        ids_dev = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
        w_dev = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
        rows = [0, M // 2, M - 1]
        ref = _oracle_rows(cfg, layer, hidden, ids_dev, w_dev, rows)
        util.assert_output_close(out[rows].float().cpu().numpy(), ref)
    # the streaming GEMV path refuses the shape instead of running past its limits
    import sm120_moe_bench_b200._lib as L
    with pytest.raises(L.VmoeError):
        vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, 4, has_shared=True, path=GEMV))


@pytest.mark.parametrize("path", PATHS)
def test_non_finite_router_logits_are_safe(vm, path):
    """Rows with a NaN, +inf or all -inf logit: the reference's router leaves their ids at -1
    (fused-moe/csrc/megakernel_v1.cu:516-528); here they get valid, distinct ids (what oracle.moe.route pins), so
    nothing indexes out of range, their output rows are NaN, and every other row is untouched by them."""
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.LayerConfig("mid", 512, 256, 12, 3, True)
    layer = synth.make_layer(cfg, seed=3)
    routed, shared = _device_layer(vm, layer)
    M = 9
    hidden, logits = synth.make_inputs(cfg, M, seed=77)
    clean = logits.clone()
    logits[1, 4] = float("nan")
    logits[4, 0] = float("inf")
    logits[6, :] = float("-inf")
    ids_ref, w_ref = omoe.route(logits.numpy(), cfg.topk)
    ids, w = ops.route(logits.cuda(), cfg.topk)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert np.array_equal(np.isnan(w.cpu().numpy()), np.isnan(w_ref))
    for m in (1, 4, 6):
        assert ids_ref[m].tolist() == [0, 1, 2] and np.isnan(w_ref[m]).all()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=path))
    out = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits.cuda(), shared=shared).clone()
    ref = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=clean.cuda(), shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    good = [0, 2, 3, 5, 7, 8]
    assert torch.equal(out[good], ref[good])
    assert torch.isnan(out[[1, 4, 6]].float()).all()


@pytest.mark.parametrize("path", PATHS)
def test_out_of_range_expert_ids_are_dropped_and_reported(vm, path):
    """Pre-routed ids outside [0, E) never index anything: the pair is dropped; an id past the range also sets
    VMOE_ERR_LIMIT in the status word.  Negative ids (a framework's "no expert" marker) drop silently."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.LayerConfig("mid", 512, 256, 12, 3, False)
    layer = synth.make_layer(cfg, seed=3)
    routed, _ = _device_layer(vm, layer)
    M = 6
    hidden, logits = synth.make_inputs(cfg, M, seed=5)
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, path=path))
    bad = ids.copy()
    bad[2, 1] = -1
    keep = np.ones_like(w); keep[2, 1] = 0
    out = vm.fused_moe(hidden.cuda(), routed, ws, topk_ids=torch.from_numpy(bad).cuda(), topk_weights=torch.from_numpy(w).cuda())
    torch.cuda.synchronize()
    assert ws.status() == 0
    ok_ids = ids.copy()
    ref = omoe.moe_layer(hidden.float().numpy(), ok_ids, (w * keep).astype(np.float32), util.to_oracle_weights(layer["routed"]))
    util.assert_output_close(out.float().cpu().numpy(), ref)
    bad[4, 0] = 1 << 20
    keep[4, 0] = 0
    out = vm.fused_moe(hidden.cuda(), routed, ws, topk_ids=torch.from_numpy(bad).cuda(), topk_weights=torch.from_numpy(w).cuda())
    torch.cuda.synchronize()
    assert ws.status() == 8                  # VMOE_ERR_LIMIT; the read clears the word
    assert ws.status() == 0
    ref = omoe.moe_layer(hidden.float().numpy(), ok_ids, (w * keep).astype(np.float32), util.to_oracle_weights(layer["routed"]))
    util.assert_output_close(out.float().cpu().numpy(), ref)


def test_checkpoint_layer_runs_on_the_device(vm, tmp_path):
    """A layer written in checkpoint naming (per-expert gate_proj / up_proj / down_proj .weight, .weight_scale,
    .weight_scale_2, as fused-moe/ep_moe_poc.py:26-57 reads them), loaded by checkpoint.load_moe_layer and run
    through fused_moe on the tensor-core path, against the oracle on the original tensors."""
    from sm120_moe_bench_b200 import checkpoint, ops, synth
    cfg = synth.LayerConfig("ckpt", 512, 256, 6, 2, True)
    layer = synth.make_layer(cfg, seed=13)
    checkpoint.save_moe_layer(str(tmp_path), 3, layer["routed"], layer["shared"], shards=2)
    loaded = checkpoint.load_moe_layer(str(tmp_path), 3, cfg.num_experts, shared_prefix=checkpoint.DEFAULT_SHARED_PREFIX)
    routed = ops.MoEWeights(*[t.cuda() for t in loaded["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in loaded["shared"]]).prepare()
    M = 7
    hidden, logits = synth.make_inputs(cfg, M, seed=2)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=TC))
    out = vm.fused_moe(hidden.cuda(), routed, ws, router_logits=logits.cuda(), shared=shared)
    torch.cuda.synchronize()
    assert ws.status() == 0
    ids, _ = omoe.route(logits.numpy(), cfg.topk)
    w_dev = ws.view("topk_weights", torch.float32, M * cfg.topk).cpu().numpy().reshape(M, cfg.topk)
    ref = omoe.moe_layer(hidden.float().numpy(), ids, w_dev, util.to_oracle_weights(layer["routed"]),
                         util.to_oracle_weights(layer["shared"]))
    util.assert_output_close(out.float().cpu().numpy(), ref)


def test_expert_parallel_halves_sum_to_whole(vm):
    """a4: two ranks each holding half of the experts (expert_map with -1 for the other half); the
    fp32 sum of their outputs equals the single-GPU output up to one bf16 rounding per rank."""
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.LayerConfig("ep", 1024, 512, 16, 4, False)
    layer = synth.make_layer(cfg, seed=9)
    hidden, logits = synth.make_inputs(cfg, 24, seed=2)
    routed, _ = _device_layer(vm, layer)
    hid_d, log_d = hidden.cuda(), logits.cuda()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, 16, cfg.topk, 24))
    full = vm.fused_moe(hid_d, routed, ws, router_logits=log_d).float()
    parts = []
    for r in range(2):
        emap = torch.full((16,), -1, dtype=torch.int32)
        emap[r * 8:(r + 1) * 8] = torch.arange(8, dtype=torch.int32)
        half = ops.MoEWeights(*[t[r * 8:(r + 1) * 8].contiguous().cuda() for t in layer["routed"]])
        wsr = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, 8, cfg.topk, 24, num_global_experts=16))
        parts.append(vm.fused_moe(hid_d, half, wsr, router_logits=log_d, expert_map=emap.cuda()).float())
    torch.cuda.synchronize()
    err = (parts[0] + parts[1] - full).abs().max().item()
    assert err <= 2 ** -7 * full.abs().max().item()


def test_back_to_back_calls_of_different_sizes_do_not_interfere(vm):
    """Calls are queued without synchronisation, alternating batch sizes (and with them the one-CTA front, the
    weights-as-rows kernel with its in-kernel combine and the token-major kernels) over ONE workspace.  The kernels of consecutive calls overlap
    their prologues (programmatic dependent launch), so each result is compared with the same call made
    alone: bit-identical."""
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.LayerConfig("mid", 512, 256, 12, 3, True)
    layer = synth.make_layer(cfg, seed=5)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare()
    sizes = [64, 1, 300, 7, 150, 2, 300, 33]
    Mmax = max(sizes)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, Mmax, has_shared=True, path=2))
    inputs = [tuple(t.cuda() for t in synth.make_inputs(cfg, M, seed=100 + i)) for i, M in enumerate(sizes)]
    alone = []
    for h, l in inputs:
        alone.append(vm.fused_moe(h, routed, ws, router_logits=l, shared=shared).clone())
        torch.cuda.synchronize()
    for rep in range(3):
        outs = [torch.empty_like(h) for h, _ in inputs]
        for (h, l), o in zip(inputs, outs):
            vm.fused_moe(h, routed, ws, router_logits=l, shared=shared, out=o)        # no synchronisation in between
        torch.cuda.synchronize()
        for o, a in zip(outs, alone):
            assert torch.equal(o, a)
    assert ws.status() == 0

