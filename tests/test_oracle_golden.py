"""The CPU oracle against vectors produced by the reference's own Python helpers
(tests/golden/make_golden.py) and against the known-answer anchors in its sources."""
import numpy as np

from oracle import moe, nvfp4


def test_e4m3_anchors():
    # fused-moe/csrc/collective_mma_test.cu:9 and gemm2_test.cu:18: 0x38 is 1.0; max finite 448
    assert nvfp4.e4m3_decode(np.array([0x38], np.uint8))[0] == 1.0
    assert nvfp4.e4m3_decode(np.array([0x7E], np.uint8))[0] == 448.0
    assert nvfp4.e4m3_encode(np.array([1.0, 448.0, 1e9], np.float32)).tolist() == [0x38, 0x7E, 0x7E]
    # device decode: NaN patterns read as zero (…tma_ext.cu:48-55)
    assert nvfp4.e4m3_decode(np.array([0x7F, 0xFF], np.uint8)).tolist() == [0.0, 0.0]
    # sub-normals m * 2**-9
    assert nvfp4.e4m3_decode(np.array([1, 7], np.uint8)).tolist() == [2.0 ** -9, 7 * 2.0 ** -9]


def test_e4m3_roundtrip_all_bytes():
    b = np.arange(256, dtype=np.uint8)
    finite = (b & 0x7F) != 0x7F
    v = nvfp4.e4m3_decode(b)
    assert np.array_equal(nvfp4.e4m3_encode(v[finite]), b[finite])


def test_e2m1_grid_on_table(golden):
    # fused-moe/tests/test_gemm1_swiglu.py:102-111: values on the E2M1 grid survive
    x = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -1.0, -3.0], np.float32)
    for tie in ("away", "low"):
        assert np.array_equal(nvfp4.e2m1_decode(nvfp4.e2m1_encode(x, tie)), x)


def test_e2m1_encoder_vs_reference_python(golden):
    grid = golden["e2m1_grid"]
    ref = golden["e2m1_codes_ref"]
    # the reference's python encoder keeps the lower code on a tie and encodes -0.0 / 0 as sign 0
    got = nvfp4.e2m1_encode(grid, tie="low")
    assert np.array_equal(got, ref)
    # the device rule differs from it exactly on the seven thresholds (both signs)
    away = nvfp4.e2m1_encode(grid, tie="away")
    diff = np.nonzero(away != ref)[0]
    assert set(np.abs(grid[diff]).tolist()) == {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0}
    assert np.all((away[diff] & 7) == (ref[diff] & 7) + 1)


def test_quantize_vs_reference_python(golden):
    x = golden["q1_in"]
    packed, sf = nvfp4.quantize_act(x, tie="low", floor=1e-12)
    assert np.array_equal(sf, golden["q1_sf"])
    assert np.array_equal(packed, golden["q1_packed"])


def test_dequant_vs_reference_python(golden):
    shape = golden["q1_in"].shape
    d = nvfp4.dequantize(golden["q1_packed"], golden["q1_sf"]).reshape(shape)
    assert np.array_equal(d, golden["q1_deq"])
    d = nvfp4.dequantize(golden["q1_packed"], golden["q1_sf"], 0.375).reshape(shape)
    assert np.array_equal(d, golden["q1_deq_alpha"])


def test_dequant_global_scale_vs_reference(golden):
    d = nvfp4.dequantize(golden["gs_packed"], golden["gs_sf"], golden["gs_scale"])
    assert np.array_equal(nvfp4.bf16_round(d), golden["gs_deq_bf16_as_f32"])


def test_cutedsl_helpers(golden):
    if "cd_a" not in golden.files:
        import pytest
        pytest.skip("vectors were generated without the DSL module")
    for name in ("a", "b"):
        packed, sf = nvfp4.quantize_act(golden["cd_" + name], tie="low", floor=1e-12 / 6.0)
        assert np.array_equal(sf, golden[f"cd_{name}_sf"])
        assert np.array_equal(packed, golden[f"cd_{name}_packed"])
    a_deq = nvfp4.dequantize(golden["cd_a_packed"], golden["cd_a_sf"])
    b_deq = nvfp4.dequantize(golden["cd_b_packed"], golden["cd_b_sf"])
    assert np.array_equal(a_deq, golden["cd_a_deq"])
    np.testing.assert_allclose(a_deq.astype(np.float64) @ b_deq.astype(np.float64).T,
                               golden["cd_c"], rtol=1e-5, atol=1e-5)


def test_known_answer_layer(golden):
    """fused-moe/test_verdict_moe_ext.py:126-218: M=1, K=256, N_half=32, 3 experts, router
    weights 1/3, seed 42 -- weights quantised by the reference, layer math redone with the
    oracle's primitives (scalar-path variant: bf16 activations, E4M3 value round trip of the
    intermediate)."""
    E, N_half = 3, 32
    packed, sf = nvfp4.quantize_act(golden["kat_w1_float"], tie="low", floor=1e-12)
    assert np.array_equal(packed, golden["kat_w1_fp4"]) and np.array_equal(sf, golden["kat_w1_sf"])
    packed, sf = nvfp4.quantize_act(golden["kat_w2_float"], tie="low", floor=1e-12)
    assert np.array_equal(packed, golden["kat_w2_fp4"]) and np.array_equal(sf, golden["kat_w2_sf"])
    x = golden["kat_input"]
    out = np.zeros_like(golden["kat_out"])
    for e in range(E):
        w1 = nvfp4.dequantize(golden["kat_w1_fp4"][e], golden["kat_w1_sf"][e])
        w2 = nvfp4.dequantize(golden["kat_w2_fp4"][e], golden["kat_w2_sf"][e])
        g1 = (x.astype(np.float64) @ w1.astype(np.float64).T).astype(np.float32)
        s = (g1[:, N_half:] * moe.silu(g1[:, :N_half])).astype(np.float32)
        inter = nvfp4.e4m3_decode(nvfp4.e4m3_encode(np.clip(s, -448, 448)))
        # the E4M3 round trip is discontinuous: allow a handful of one-step differences
        ref_inter = golden["kat_inter_e4m3"][e]
        assert np.mean(inter != ref_inter) <= 0.05
        np.testing.assert_allclose(inter, ref_inter, rtol=0.13, atol=2.0 ** -9)
        out += np.float32(1.0 / 3.0) * (ref_inter.astype(np.float64) @ w2.astype(np.float64).T).astype(np.float32)
    err = np.abs(out - golden["kat_out"]).mean() / np.abs(golden["kat_out"]).mean()
    assert err < 1e-5, err
