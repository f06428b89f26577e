"""Helpers shared by the parity tests: synthetic layers as both torch (device) and numpy (oracle)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import moe as omoe
from oracle import nvfp4


def to_oracle_weights(six, experts=None) -> omoe.ExpertWeights:
    """6-tuple of torch tensors -> oracle ExpertWeights (optionally only some experts, others zero-sized
    views are avoided by keeping the expert axis and copying just the selected rows)."""
    w13, w13_sf, w13_gs, w2, w2_sf, w2_gs = six
    if experts is None:
        conv = lambda t: t.cpu().numpy()
        return omoe.ExpertWeights(conv(w13), conv(w13_sf), conv(w13_gs), conv(w2), conv(w2_sf), conv(w2_gs))
    E = w13.shape[0]
    idx = torch.as_tensor(sorted(set(int(e) for e in experts)), device=w13.device)

    class Sparse:
        """expert-indexed view that only holds the requested experts"""
        def __init__(self, t):
            self.shape = t.shape
            self.data = {int(e): t[int(e)].cpu().numpy() for e in idx}
        def __getitem__(self, e):
            return self.data[int(e)]
    return omoe.ExpertWeights(Sparse(w13), Sparse(w13_sf), w13_gs.cpu().numpy(),
                              Sparse(w2), Sparse(w2_sf), w2_gs.cpu().numpy())


def bf16_to_f32_numpy(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) /
                 max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel(); b = b.astype(np.float64).ravel()
    return float(a @ b / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-30))


# Output tolerance of the fused layer against the fp32 (f64-accumulated) oracle.  The only
# sources of difference are fp32 accumulation order in the two GEMMs, a last-bit difference in
# expf, and the (rare) E2M1 / E4M3 code flips of the re-quantised intermediate these cause.
OUT_COSINE_MIN = 0.9999
OUT_REL_L2_MAX = 5e-3
OUT_MAX_ABS_FRAC = 1e-2      # max |diff| <= this * max |ref|
INTER_FLIP_RATE_MAX = 2e-3   # fraction of intermediate FP4 codes allowed to differ


def assert_output_close(got: np.ndarray, ref: np.ndarray):
    c, r = cosine(got, ref), rel_l2(got, ref)
    ma = float(np.max(np.abs(got - ref))) / max(float(np.max(np.abs(ref))), 1e-30)
    assert c >= OUT_COSINE_MIN and r <= OUT_REL_L2_MAX and ma <= OUT_MAX_ABS_FRAC, (c, r, ma)
    return c, r, ma
