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
