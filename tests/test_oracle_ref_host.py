"""The oracle against the reference's own host C++ reference, compiled from the reference checkout by
``oracle/build_ref.py`` into ``oracle/_ref/libref_host.so`` (fused-moe/csrc/verdict_fused_independent.cu:50-86,
474-564).  Skipped where that library has not been built.  No GPU is used: only host functions run."""
import numpy as np
import pytest

from oracle import moe as omoe
from oracle import nvfp4, ref_host

ref = ref_host.load()
pytestmark = pytest.mark.skipif(ref is None, reason="oracle/_ref/libref_host.so has not been built")


def test_e4m3_decode_all_bytes():
    got = ref.e4m3_decode_all()
    want = nvfp4.e4m3_decode(np.arange(256, dtype=np.uint8), nan_to_zero=False)   # the host rule keeps NaN
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(got)
    assert np.array_equal(got[ok], want[ok])
    # device rule: the two NaN patterns decode to zero, everything else is the same
    dev = nvfp4.e4m3_decode(np.arange(256, dtype=np.uint8))
    assert np.array_equal(dev[ok], got[ok]) and dev[0x7F] == 0 and dev[0xFF] == 0


def test_e4m3_encoders():
    g = np.random.default_rng(0)
    x = np.concatenate([np.exp(g.uniform(np.log(1e-4), np.log(600.0), 4000)).astype(np.float32),
                        nvfp4.e4m3_decode(np.arange(0x7F, dtype=np.uint8)),          # exactly representable
                        np.array([0.0, -1.0, 448.0, 449.0, 1e-30, 2.0 ** -9, 2.0 ** -10], np.float32)])
    assert np.array_equal(ref.e4m3_encode_ceil(x), nvfp4.e4m3_encode_ceil(x))
    # nearest encoders: the host search and round-to-nearest-even agree off the exact midpoints
    pos = x[(x > 0) & (x < 448)]
    vals = nvfp4.e4m3_decode(np.arange(0x7F, dtype=np.uint8))
    mids = (vals[1:] + vals[:-1]) / 2
    off_mid = pos[~np.isin(pos, mids)]
    assert np.array_equal(ref.e4m3_encode(off_mid), nvfp4.e4m3_encode(off_mid))


def test_block_quantiser_bit_exact():
    g = np.random.default_rng(1)
    for scale in (1.0, 1e-3, 50.0):
        data = (g.standard_normal(16 * 300) * scale).astype(np.float32)
        rp, rs = ref.quantize(data)
        op, osf = nvfp4.quantize_act(data.reshape(1, -1), tie="low", scale_round="ceil")
        assert np.array_equal(rs, osf.ravel())
        assert np.array_equal(rp, op.ravel())
        # and the decoder
        assert np.array_equal(ref.dequantize(rp[:64], rs[:8]), nvfp4.dequantize(op[:, :64], osf[:, :8]).ravel())
    # what differs from the device rule: block scales rounded up instead of to nearest
    data = (g.standard_normal(16 * 300)).astype(np.float32)
    _, sf_dev = nvfp4.quantize_act(data.reshape(1, -1))
    _, sf_host = ref.quantize(data)
    assert (sf_host >= sf_dev.ravel()).all() and (sf_host != sf_dev.ravel()).any()


def test_layer_single_token():
    """host_quantized_reference_single (hidden 4096, no global scales) against the oracle's expert pipeline run
    with the harness's quantiser rules: same intermediate codes, output within fp32 summation-order noise."""
    from sm120_moe_bench_b200 import synth
    import torch
    K, N, E = ref.hidden, 256, 4
    gen = torch.Generator().manual_seed(5)
    w13, w13_sf, _, w2, w2_sf, _ = (t.numpy() for t in synth.make_expert_weights(E, K, N, gen, "cpu"))
    ones = np.ones(E, np.float32)
    ew = omoe.ExpertWeights(w13, w13_sf, ones, w2, w2_sf, ones)
    g = np.random.default_rng(2)
    x = g.standard_normal(K).astype(np.float32)
    xp, xs = ref.quantize(x)
    ids = np.array([2, 0, 3], np.int32); wts = np.array([0.5, 0.3, 0.2], np.float32)
    got = ref.layer_single(xp, xs, w13, w13_sf, w2, w2_sf, ids, wts)
    want = np.zeros(K, np.float64)
    for e, wt in zip(ids, wts):
        y, s_packed, s_sf, s = omoe.expert_mlp(xp.reshape(1, -1), xs.reshape(1, -1), ew, int(e), accum="f64",
                                               return_inter=True, requant=dict(tie="low", scale_round="ceil"))
        want += float(wt) * y[0].astype(np.float64)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel < 2e-4, rel
    cos = float(np.dot(got, want) / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert cos > 0.99999


# ---------------------------------------------------------------------------------------------
# Router and permutation against the reference's own functions (compiled by oracle/build_ref.py)
# ---------------------------------------------------------------------------------------------
ref_router = ref_host.load_router()
ref_tables = ref_host.load_tables()


def _config_logits():
    from sm120_moe_bench_b200 import synth
    out = []
    for cfg, M, zipf in ((synth.CONFIG_TINY, 4, None), (synth.CONFIG_LARGE, 64, None), (synth.CONFIG_LARGE, 64, 1.2)):
        _, logits = synth.make_inputs(cfg, M, seed=0, zipf_s=zipf)
        out.append((cfg, logits.numpy()))
    return out


@pytest.mark.skipif(ref_router is None, reason="oracle/_ref/libref_router.so has not been built")
def test_route_matches_reference_topk_select():
    """oracle.moe.route against moe_topk_select (fused-moe/csrc/megakernel_v1.cu:491-537) on the logits of
    BASELINE configs 1 and 2 (uniform and Zipf): ids and their order bit for bit, weights to the last bits of
    two different expf implementations; plus exact ties (lowest id first)."""
    for cfg, logits in _config_logits():
        ids, w = omoe.route(logits, cfg.topk)
        rid, rw = ref_router.route(logits, cfg.topk)
        assert omoe.route_ids_are_unambiguous(logits, cfg.topk)
        assert np.array_equal(ids, rid)
        assert np.allclose(w, rw, rtol=2e-6, atol=0)
    tie = np.zeros((2, 16), np.float32)
    tie[1, [3, 9, 12]] = 1.0
    ids, w = omoe.route(tie, 4)
    rid, rw = ref_router.route(tie, 4)
    assert np.array_equal(ids, rid) and ids[0].tolist() == [0, 1, 2, 3] and ids[1].tolist() == [3, 9, 12, 0]
    assert np.allclose(w, rw, rtol=2e-6, atol=0)


@pytest.mark.skipif(ref_router is None, reason="oracle/_ref/libref_router.so has not been built")
def test_route_non_finite_rows_are_pinned_differently_from_the_reference():
    """The reference leaves ids at -1 for a row whose softmax is NaN; the oracle (and the device) pin valid
    ids and NaN weights instead.  This test records both behaviours."""
    lg = np.random.default_rng(0).standard_normal((3, 32)).astype(np.float32)
    lg[0, 5] = np.nan
    lg[1, 7] = np.inf
    rid, _ = ref_router.route(lg, 4)
    assert (rid[0] == -1).all() and (rid[1] == -1).all()
    ids, w = omoe.route(lg, 4)
    assert ids[0].tolist() == [0, 1, 2, 3] and ids[1].tolist() == [0, 1, 2, 3]
    assert np.isnan(w[0]).all() and np.isnan(w[1]).all()
    assert np.array_equal(ids[2], rid[2]) and np.isfinite(w[2]).all()


@pytest.mark.skipif(ref_tables is None, reason="oracle/_ref/libref_tables.so has not been built")
def test_group_tables_match_reference_build_group_tables():
    """oracle.moe.build_group_tables against build_group_tables (fused-moe/csrc/verdict_fused_grouped.cu:655-691)
    on the routing of BASELINE configs 1 and 2 and on a ragged random case: every table bit for bit."""
    cases = [(omoe.route(lg, cfg.topk)[0], cfg.num_experts) for cfg, lg in _config_logits()]
    rng = np.random.default_rng(3)
    cases.append((np.stack([rng.permutation(40)[:7] for _ in range(37)]).astype(np.int32), 40))
    cases.append((np.zeros((1, 1), np.int32), 4))
    for ids, E in cases:
        w = np.full(ids.shape, 0.25, np.float32)
        t = omoe.build_group_tables(ids, w, E)
        r = ref_tables.build_group_tables(ids, 0.25)
        assert np.array_equal(t.expert_list, r["expert_list"])
        assert np.array_equal(t.expert_token_count, r["expert_token_count"])
        assert np.array_equal(t.expert_token_offset, r["expert_token_offset"])
        assert np.array_equal(t.gather_idx, r["gather_idx"])
        assert np.array_equal(t.scatter_weights, r["scatter_weights"])
