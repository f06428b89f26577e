#!/usr/bin/env python3
"""Generate ``tests/golden/ref_vectors.npz`` by running the reference project's own
pure-torch helpers on seeded inputs.

Run once, in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/reference

The reference functions that are imported and executed (unmodified):

* ``fused-moe/test_verdict_moe_ext.py``: ``quantize_nvfp4`` (:62-100),
  ``dequant_nvfp4_ref`` (:103-123), ``encode_fp4_e2m1`` (:47-59), and the
  per-expert reference loop of ``test_correctness`` (:196-218), which is inline
  in a function that needs a GPU and is therefore re-run here statement by
  statement on CPU tensors with the imported helpers;
* ``fused-moe/ep_moe_poc.py``: ``dequant_nvfp4`` with a global scale (:60-98);
* ``fused-moe/verdict_moe/test_gemm_cutedsl.py``: ``nvfp4_quantize`` (:26-68),
  ``nvfp4_dequantize`` (:71-97), ``reference_gemm`` (:100-102) -- only if the
  module's DSL imports succeed.

The resulting file is small (tens of KB) and is committed; the tests never
read the reference project itself.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str):
    ref = Path(ref_root)
    out = {}
    tv = _load(ref / "fused-moe" / "test_verdict_moe_ext.py", "ref_test_verdict_moe_ext")
    ep = _load(ref / "fused-moe" / "ep_moe_poc.py", "ref_ep_moe_poc")

    # ---- (1) quantize_nvfp4 / dequant_nvfp4_ref on seeded tensors -------------
    torch.manual_seed(42)
    x = torch.randn(6, 8, 64) * (2.0 / 8.0)
    x[0, 0, :16] = 0.0                       # an all-zero block
    x[1, 1, 3] = 37.5                        # a large outlier
    packed, sf = tv.quantize_nvfp4(x)
    out["q1_in"] = x.numpy()
    out["q1_packed"] = packed.numpy()
    out["q1_sf"] = sf.numpy()
    out["q1_deq"] = tv.dequant_nvfp4_ref(packed, sf, 1.0, tuple(x.shape)).numpy()
    out["q1_deq_alpha"] = tv.dequant_nvfp4_ref(packed, sf, 0.375, tuple(x.shape)).numpy()

    # E2M1 scalar encoder over a grid that includes every threshold
    grid = np.concatenate([np.linspace(-7, 7, 561, dtype=np.float32),
                           np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32),
                           -np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)])
    out["e2m1_grid"] = grid
    out["e2m1_codes_ref"] = np.array([tv.encode_fp4_e2m1(float(v)) for v in grid], np.uint8)

    # ---- (2) the published known-answer configuration: M=1, K=256, N_half=32,
    #          3 experts, weights randn*2/sqrt(fan_in), router weights 1/3, seed 42
    torch.manual_seed(42)
    M, K, N_half, E = 1, 256, 32, 3
    N2 = 2 * N_half
    w1_float = torch.randn(E, N2, K) * (2.0 / (K ** 0.5))
    w2_float = torch.randn(E, K, N_half) * (2.0 / (N_half ** 0.5))
    input_f32 = torch.randn(M, K, dtype=torch.bfloat16).float()
    w1_fp4, w1_sf = tv.quantize_nvfp4(w1_float)
    w2_fp4, w2_sf = tv.quantize_nvfp4(w2_float)
    w1_deq = tv.dequant_nvfp4_ref(w1_fp4, w1_sf, 1.0, (E, N2, K))
    w2_deq = tv.dequant_nvfp4_ref(w2_fp4, w2_sf, 1.0, (E, K, N_half))
    wts = torch.ones(E) / E
    ref_out = torch.zeros(M, K)
    inter_all = []
    for e in range(E):
        gemm1 = input_f32 @ w1_deq[e].T
        gate = gemm1[:, :N_half]
        up = gemm1[:, N_half:]
        swiglu = gate * torch.sigmoid(gate) * up
        inter = swiglu.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
        inter_all.append(inter.numpy())
        ref_out += wts[e].item() * (inter @ w2_deq[e].T)
    out["kat_w1_float"] = w1_float.numpy()
    out["kat_w2_float"] = w2_float.numpy()
    out["kat_input"] = input_f32.numpy()
    out["kat_w1_fp4"] = w1_fp4.numpy()
    out["kat_w1_sf"] = w1_sf.numpy()
    out["kat_w2_fp4"] = w2_fp4.numpy()
    out["kat_w2_sf"] = w2_sf.numpy()
    out["kat_inter_e4m3"] = np.stack(inter_all)
    out["kat_out"] = ref_out.numpy()

    # ---- (3) dequant with a global scale ---------------------------------------
    torch.manual_seed(7)
    pk = torch.randint(0, 256, (12, 32), dtype=torch.uint8)
    sc_bytes = torch.randint(0, 0x7F, (12, 4), dtype=torch.uint8)   # no NaN pattern
    gs = torch.tensor(0.00123, dtype=torch.float32)
    deq = ep.dequant_nvfp4(pk, sc_bytes.view(torch.float8_e4m3fn), gs, 12, 64)
    out["gs_packed"] = pk.numpy()
    out["gs_sf"] = sc_bytes.numpy()
    out["gs_scale"] = np.float32(gs.item())
    out["gs_deq_bf16_as_f32"] = deq.float().numpy()

    # ---- (4) the DSL test module's torch helpers (optional) ----------------------
    try:
        cd = _load(ref / "fused-moe" / "verdict_moe" / "test_gemm_cutedsl.py", "ref_test_gemm_cutedsl")
        torch.manual_seed(42)
        a = torch.randn(4, 64) * 0.5
        b = torch.randn(16, 64) * 0.5
        ap, asf = cd.nvfp4_quantize(a, 16)
        bp, bsf = cd.nvfp4_quantize(b, 16)
        out["cd_a"] = a.numpy()
        out["cd_b"] = b.numpy()
        out["cd_a_packed"] = ap.numpy()
        out["cd_a_sf"] = asf.view(torch.uint8).numpy()
        out["cd_b_packed"] = bp.numpy()
        out["cd_b_sf"] = bsf.view(torch.uint8).numpy()
        a_deq = cd.nvfp4_dequantize(ap, asf, 16)
        b_deq = cd.nvfp4_dequantize(bp, bsf, 16)
        out["cd_a_deq"] = a_deq.numpy()
        out["cd_c"] = cd.reference_gemm(a_deq, b_deq).numpy()
        print("cutedsl helpers: included")
    except Exception as exc:  # DSL import not available: vectors simply absent
        print("cutedsl helpers: skipped (%s: %s)" % (type(exc).__name__, exc))

    dst = Path(__file__).parent / "ref_vectors.npz"
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("VMOE_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py <reference checkout>   (or set VMOE_REFERENCE_ROOT)")
    main(root)
