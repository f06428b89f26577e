"""CPU oracle, part 1: the NVFP4 codec (E2M1 values, E4M3 block scales).

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product:
only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import it, and only as the checker.

Every function restates, in numpy, arithmetic that the reference performs in
the files cited in its docstring (paths are relative to the reference
project's root).  Where the reference is inconsistent with itself, the rule of
its *device* code is the pinned one and the alternative is available through
an argument so that the Python helpers of the reference can be reproduced bit
for bit as well (see ``tests/golden/make_golden.py``).

Parity is pinned: ``tests/test_oracle_golden.py`` checks these functions
against vectors produced by importing the reference's own Python helpers.
"""
from __future__ import annotations

import numpy as np

# fused-moe/csrc/verdict_moe_ext.cu:36-38 and
# fused-moe/csrc/verdict_fused_independent.cu:45 -- the eight E2M1 magnitudes.
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)

# fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:68-76 -- the seven
# decision thresholds; a value is compared with ``<`` so a magnitude that sits
# exactly on a threshold takes the larger code (ties go away from zero).
E2M1_THRESHOLDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)

SF_BLOCK = 16  # elements covered by one E4M3 block scale


# --------------------------------------------------------------------------
# E4M3 (fn: no infinities, 0x7F / 0xFF are NaN)
# --------------------------------------------------------------------------
def e4m3_decode(b: np.ndarray, nan_to_zero: bool = True) -> np.ndarray:
    """Decode E4M3FN bytes to float32.

    fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:48-55: sub-normals are
    ``m * 2**-9``, normals ``(8 + m) * 2**(e - 10)``, the sign bit is honoured,
    and the NaN patterns 0x7F / 0xFF decode to **0.0** on the device.  The host
    harness (fused-moe/csrc/verdict_fused_independent.cu:50-55) returns NaN for
    them instead; ``nan_to_zero=False`` gives that behaviour.
    """
    b = np.asarray(b, dtype=np.uint8)
    s = (b >> 7) & 1
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 7).astype(np.float32)
    sub = np.ldexp(m, -9).astype(np.float32)
    nor = np.ldexp(np.float32(8.0) + m, e - 10).astype(np.float32)
    val = np.where(e == 0, sub, nor).astype(np.float32)
    is_nan = (e == 15) & ((b & 7) == 7)
    val = np.where(is_nan, np.float32(0.0 if nan_to_zero else np.nan), val)
    return np.where(s == 1, -val, val).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3FN byte, round-to-nearest-even, saturating at +-448.

    This is ``cvt.rn.satfinite.e4m3x2.f32`` as the reference's device code
    uses it (fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:57-62): RNE,
    every finite magnitude above 448 (and +-inf) becomes 0x7E / 0xFE, NaN
    becomes 0x7F.  It is *not* the round-up encoder of the host harness
    (fused-moe/csrc/verdict_fused_independent.cu:73-84).
    """
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x).astype(np.uint8) << 7
    a = np.abs(x)
    nan = np.isnan(a)
    a = np.where(nan, np.float32(0.0), a)
    a = np.minimum(a, np.float32(448.0))
    # sub-normal range (below 2**-6): the byte is round(a * 2**9) in 0..8
    # (8 is the smallest normal, 0x08, so the carry falls out by itself).
    sub = np.rint(a * np.float32(512.0)).astype(np.int32)
    # normal range: a = f * 2**ex, f in [0.5, 1)
    _, ex = np.frexp(np.maximum(a, np.float32(2.0 ** -6)))
    ex = ex.astype(np.int32) - 1                      # a in [2**ex, 2**(ex+1))
    q = np.rint(np.ldexp(a, 3 - ex)).astype(np.int32)  # in 8..16, exact scaling
    carry = q == 16
    ex = np.where(carry, ex + 1, ex)
    q = np.where(carry, 8, q)
    nor = ((ex + 7) << 3) | (q - 8)
    byte = np.where(a < np.float32(2.0 ** -6), sub, nor)
    byte = np.minimum(byte, 0x7E).astype(np.uint8)
    byte = np.where(nan, np.uint8(0x7F), byte | sign)
    return byte.astype(np.uint8)


def e4m3_encode_ceil(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3FN byte, rounded UP to the next representable magnitude: the block-scale encoder of the
    reference's host harness (fused-moe/csrc/verdict_fused_independent.cu:73-84): ``x <= 0`` gives 0x08,
    ``x >= 448`` gives 0x7E, otherwise the smallest representable value that is ``>= x``.  The device code
    rounds to nearest instead (``e4m3_encode``); this variant exists to check the oracle against the compiled
    host reference."""
    x = np.asarray(x, dtype=np.float32)
    codes = np.arange(0x7F, dtype=np.uint8)                      # 0x00 .. 0x7E, ascending values
    values = e4m3_decode(codes)
    idx = np.searchsorted(values, x, side="left")
    idx = np.clip(idx, 0, 0x7E)
    out = codes[idx]
    out = np.where(x <= 0, np.uint8(0x08), out)
    out = np.where(x >= np.float32(448.0), np.uint8(0x7E), out)
    return out.astype(np.uint8)


# --------------------------------------------------------------------------
# E2M1
# --------------------------------------------------------------------------
def e2m1_decode(nib: np.ndarray) -> np.ndarray:
    """4-bit code (sign<<3 | index) -> float32.
    fused-moe/csrc/verdict_moe_ext.cu:36-38,103-116."""
    nib = np.asarray(nib, dtype=np.uint8)
    mag = E2M1_VALUES[nib & 7]
    return np.where((nib >> 3) & 1, -mag, mag).astype(np.float32)


def e2m1_encode(v: np.ndarray, tie: str = "away") -> np.ndarray:
    """float32 -> 4-bit code.

    ``tie="away"`` is the device rule: index = number of thresholds that are
    <= |v| (fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:68-76), the
    sign bit is ``v < 0`` (so -0.0 and NaN give sign 0; NaN gives index 7
    because every ``<`` comparison is false).
    ``tie="low"`` is the nearest-value search of the reference's Python
    helpers, which keeps the smaller code on a tie
    (fused-moe/test_verdict_moe_ext.py:47-59,
    fused-moe/verdict_moe/test_gemm_cutedsl.py:57-58).
    """
    v = np.asarray(v, dtype=np.float32)
    av = np.abs(v)
    if tie == "away":
        idx = np.zeros(v.shape, dtype=np.uint8)
        for t in E2M1_THRESHOLDS:
            idx += (~(av < t)).astype(np.uint8)
    elif tie == "low":
        diffs = np.abs(av[..., None] - E2M1_VALUES)
        idx = np.argmin(diffs, axis=-1).astype(np.uint8)
    else:
        raise ValueError(tie)
    sign = (v < 0).astype(np.uint8)
    return ((sign << 3) | idx).astype(np.uint8)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """Even element -> low nibble, odd element -> high nibble
    (fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:274-276,
    fused-moe/csrc/verdict_moe_ext.cu:111-112)."""
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


# --------------------------------------------------------------------------
# Block quantisers
# --------------------------------------------------------------------------
def quantize_act(x: np.ndarray, tie: str = "away", floor: float = 1e-30, scale_round: str = "rne"):
    """Activation quantiser: float32 [..., K] -> (packed u8 [..., K/2], sf u8 [..., K/16]).

    fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:249-279 (prologue) and
    :426-452 (intermediate after SwiGLU): per 16 consecutive elements
    ``sf = max(amax / 6, 1e-30)`` -> E4M3 (RNE, saturating) -> decoded again,
    floored at 1e-30 -> ``code = e2m1(x / scale)``.  No global scale.  All
    arithmetic is float32 with IEEE division, as the reference compiles
    without fast-math (fused-moe/verdict_moe.py:67-76).

    ``tie="low", floor=1e-12`` reproduces the reference's Python
    ``quantize_nvfp4`` (fused-moe/test_verdict_moe_ext.py:62-100) for inputs
    whose block scales stay below 448.  ``tie="low", scale_round="ceil"`` reproduces the
    host harness ``quantize_to_nvfp4_e4m3`` (fused-moe/csrc/verdict_fused_independent.cu:474-496).
    """
    x = np.asarray(x, dtype=np.float32)
    K = x.shape[-1]
    assert K % SF_BLOCK == 0
    blocks = x.reshape(x.shape[:-1] + (K // SF_BLOCK, SF_BLOCK))
    with np.errstate(invalid="ignore"):
        amax = np.max(np.abs(blocks), axis=-1)
    sf_target = np.maximum(amax / np.float32(6.0), np.float32(floor)).astype(np.float32)
    if scale_round == "rne":
        sf = e4m3_encode(sf_target)
    elif scale_round == "ceil":
        sf = e4m3_encode_ceil(sf_target)
    else:
        raise ValueError(scale_round)
    scale = np.maximum(e4m3_decode(sf), np.float32(1e-30)).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = (blocks / scale[..., None]).astype(np.float32)
    codes = e2m1_encode(scaled, tie=tie).reshape(x.shape)
    return pack_nibbles(codes), sf


def quantize_weight(w: np.ndarray, global_scale=None, tie: str = "away"):
    """Synthetic-weight quantiser with an fp32 per-tensor global scale.

    The reference has no weight quantiser of its own for the global-scale form;
    it loads ``weight`` / ``weight_scale`` / ``weight_scale_2`` from a
    checkpoint and dequantises them as ``code * block_scale * global_scale``
    (fused-moe/ep_moe_poc.py:60-98).  This generator is the inverse of that
    formula: ``gs = amax / (448 * 6)``, block scale ``= e4m3(block_amax / (6 gs))``
    (saturating at 448), ``code = e2m1(w / (block_scale * gs))``.  It makes block
    scales use the top of the E4M3 range, as real checkpoints do
    (fused-moe/PHASE2_RESULTS.md:77-84).

    ``w`` is float32 ``[rows, K]``; returns ``(packed, sf, gs)`` with ``gs`` a
    float32 scalar.
    """
    w = np.asarray(w, dtype=np.float32)
    if global_scale is None:
        amax = np.float32(np.max(np.abs(w)))
        global_scale = np.float32(max(amax, np.float32(1e-30)) / np.float32(448.0 * 6.0))
    gs = np.float32(global_scale)
    K = w.shape[-1]
    blocks = w.reshape(w.shape[:-1] + (K // SF_BLOCK, SF_BLOCK))
    bmax = np.max(np.abs(blocks), axis=-1)
    sf_target = (bmax / (np.float32(6.0) * gs)).astype(np.float32)
    sf = e4m3_encode(sf_target)
    scale = (np.maximum(e4m3_decode(sf), np.float32(1e-30)) * gs).astype(np.float32)
    scaled = (blocks / scale[..., None]).astype(np.float32)
    codes = e2m1_encode(scaled, tie=tie).reshape(w.shape)
    return pack_nibbles(codes), sf, gs


def dequantize(packed: np.ndarray, sf: np.ndarray, global_scale=1.0,
               nan_to_zero: bool = True) -> np.ndarray:
    """packed u8 [..., K/2] + sf u8 [..., K/16] (+ fp32 global scale) -> float32 [..., K].

    ``value = e2m1(code) * e4m3(block_scale) * global_scale``:
    fused-moe/test_verdict_moe_ext.py:103-123, fused-moe/ep_moe_poc.py:60-98,
    fused-moe/csrc/verdict_fused_independent.cu:497-503.
    """
    vals = e2m1_decode(unpack_nibbles(packed))
    scale = e4m3_decode(sf, nan_to_zero=nan_to_zero)
    scale = np.repeat(scale, SF_BLOCK, axis=-1)
    gs = np.asarray(global_scale, dtype=np.float32)
    return (vals * scale * gs).astype(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16, returned as float32 (``__float2bfloat16``,
    fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:561)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 values that are exactly representable in bf16 -> uint16 bit patterns."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)
