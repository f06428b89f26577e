"""CPU-only checks of the oracle's routing / permutation / layer logic and of the synthetic-data
generator against it."""
import numpy as np
import torch

from oracle import moe as omoe
from oracle import nvfp4


def test_route_reference_semantics():
    """fused-moe/csrc/megakernel_v1.cu:491-537 restated literally (single thread, insertion with
    strict '>') on small inputs; the vectorised oracle must give the same ids and weights."""
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((9, 40)).astype(np.float32)
    logits[3, 7] = logits[3, 21] = logits[3].max() + 1           # exact tie for first place
    T = 6
    ids, w = omoe.route(logits, T)
    for m in range(logits.shape[0]):
        l = logits[m]
        mx = np.float32(-1e30)
        for v in l:
            mx = max(mx, v)
        p = np.exp((l - mx).astype(np.float32)).astype(np.float32)
        s = np.float32(0)
        for v in p:
            s = np.float32(s + v)
        p = (p * (np.float32(1) / s)).astype(np.float32)
        top_ids = [-1] * T; top_w = [np.float32(-1e30)] * T
        for e in range(len(p)):
            if p[e] > top_w[T - 1]:
                top_ids[T - 1] = e; top_w[T - 1] = p[e]
                j = T - 1
                while j > 0 and top_w[j] > top_w[j - 1]:
                    top_w[j], top_w[j - 1] = top_w[j - 1], top_w[j]
                    top_ids[j], top_ids[j - 1] = top_ids[j - 1], top_ids[j]
                    j -= 1
        ws = np.float32(0)
        for v in top_w:
            ws = np.float32(ws + v)
        ref_w = np.array(top_w, np.float32) * (np.float32(1) / ws)
        assert ids[m].tolist() == top_ids
        assert np.array_equal(w[m], ref_w.astype(np.float32))
    assert ids[3, :2].tolist() == [7, 21]


def test_group_tables_against_stable_sort():
    """fused-moe/csrc/verdict_fused_grouped.cu:655-691 restated with Python's stable sort."""
    rng = np.random.default_rng(1)
    M, T, E = 23, 4, 9
    ids = np.stack([rng.permutation(E)[:T] for _ in range(M)]).astype(np.int32)
    w = rng.random((M, T)).astype(np.float32)
    t = omoe.build_group_tables(ids, w, E)
    pairs = sorted([(int(ids[m, j]), m * T + j) for m in range(M) for j in range(T)], key=lambda x: x[0])
    assert t.sorted_pair.tolist() == [p for _, p in pairs]
    assert t.gather_idx.tolist() == [p // T for _, p in pairs]
    assert np.array_equal(t.scatter_weights, w.reshape(-1)[t.sorted_pair])
    assert t.expert_offsets[-1] == M * T and np.all(np.diff(t.expert_offsets) >= 0)
    assert np.array_equal(t.pair_slot[t.sorted_pair], np.arange(M * T))
    assert t.expert_token_offset[-1] == M * T
    assert np.array_equal(t.expert_list, np.unique(ids))
    # empty input
    t0 = omoe.build_group_tables(np.zeros((0, T), np.int32), np.zeros((0, T), np.float32), E)
    assert t0.sorted_pair.size == 0 and np.all(t0.expert_offsets == 0)


def test_expert_map_semantics():
    ids = np.array([[0, 5], [6, 1]], np.int32)
    w = np.array([[.6, .4], [.7, .3]], np.float32)
    emap = np.array([-1, -1, -1, -1, 0, 1, 2, 3], np.int32)
    li, lw = omoe.apply_expert_map(ids, w, emap)
    assert li.tolist() == [[0, 1], [2, 0]] and lw.tolist() == [[0.0, np.float32(.4)], [np.float32(.7), 0.0]]


def test_synth_quantiser_matches_oracle():
    from sm120_moe_bench_b200 import synth
    g = torch.Generator().manual_seed(0)
    w = torch.randn(3, 24, 128, generator=g) * 0.02
    w[1, 0, :16] = 0
    packed, sf, gs = synth.quantize_weight(w)
    for e in range(3):
        p, s, g1 = nvfp4.quantize_weight(w[e].numpy())
        assert np.float32(g1) == gs[e].item()
        assert np.array_equal(s, sf[e].numpy()) and np.array_equal(p, packed[e].numpy())
    # block scales reach the top of the E4M3 range (exponent field >= 14), as real checkpoints do
    assert (sf.numpy() >> 3).max() >= 14
    deq = nvfp4.dequantize(packed.numpy(), sf.numpy(), gs.numpy()[:, None, None])
    # worst E2M1 step is 2 (between 4 and 6): error <= 1 code unit = block amax / 6 (+ scale rounding)
    err = np.abs(deq - w.numpy()).reshape(3, 24, 8, 16).max(-1)
    bmax = np.abs(w.numpy()).reshape(3, 24, 8, 16).max(-1)
    assert np.all(err <= bmax / 6 * 1.07 + 1e-9)


def test_layer_tiny_self_consistency():
    """BASELINE config 1 on the oracle alone: f32 vs f64 accumulation agree within the layer
    tolerance, the expert-at-a-time evaluation equals a pair-at-a-time one, and expert-parallel
    halves add up to the whole."""
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_TINY
    layer = synth.make_layer(cfg, seed=0)
    hidden, logits = synth.make_inputs(cfg, 4, seed=0)
    ew = omoe.ExpertWeights(*[t.numpy() for t in layer["routed"]])
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    x = hidden.float().numpy()
    out64 = omoe.moe_layer(x, ids, w, ew, accum="f64")
    out32 = omoe.moe_layer(x, ids, w, ew, accum="f32")
    rel = np.linalg.norm(out64 - out32) / np.linalg.norm(out64)
    assert rel < 5e-3 and np.isfinite(out64).all() and np.abs(out64).max() > 0
    # pair at a time
    xq, xsf = nvfp4.quantize_act(x)
    acc = np.zeros_like(x)
    for j in range(cfg.topk):
        row = np.zeros_like(x)
        for m in range(4):
            e = int(ids[m, j])
            y = omoe.expert_mlp(xq[m:m + 1], xsf[m:m + 1], ew, e)
            row[m] = y[0] * np.float32(w[m, j] * ew.w2_gs[e])
        acc = (acc + row).astype(np.float32)
    assert np.array_equal(nvfp4.bf16_round(acc), out64)
    # expert-parallel halves
    parts = []
    for r in range(2):
        emap = np.full(8, -1, np.int32); emap[r * 4:(r + 1) * 4] = np.arange(4)
        half = omoe.ExpertWeights(*[t[r * 4:(r + 1) * 4].numpy() for t in layer["routed"]])
        parts.append(omoe.moe_layer(x, ids, w, half, expert_map=emap))
    assert np.abs(parts[0] + parts[1] - out64).max() <= 2 ** -7 * np.abs(out64).max()


def test_rmsnorm_quantize_oracle_against_float64():
    """oracle.moe.rmsnorm_quantize (fused-moe/csrc/megakernel_v1.cu:257-352 with a pinned summation order): the
    normalised rows agree with a float64 evaluation to bf16 rounding, and the codes are the activation quantiser's."""
    g = np.random.default_rng(5)
    for K in (512, 4096, 7168):
        x = nvfp4.bf16_round(g.standard_normal((4, K)).astype(np.float32) * 2.0)
        gamma = (1.0 + 0.1 * g.standard_normal(K)).astype(np.float32)
        y, packed, sf = omoe.rmsnorm_quantize(x, gamma, 1e-6)
        ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-6) * gamma
        assert np.all(np.abs(y - ref) <= np.abs(ref) * 2.0 ** -8 + 1e-6)
        assert np.array_equal(y, nvfp4.bf16_round(y))
        p2, s2 = nvfp4.quantize_act(y)
        assert np.array_equal(packed, p2) and np.array_equal(sf, s2)
    # an all-zero row stays zero and finite (eps keeps the reciprocal square root finite)
    y, packed, sf = omoe.rmsnorm_quantize(np.zeros((1, 512), np.float32), np.ones(512, np.float32), 1e-6)
    assert np.all(y == 0) and np.all(packed == 0)
