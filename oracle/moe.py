"""CPU oracle, part 2: routing, pair/permutation tables and the fused NVFP4 MoE
expert layer as dequantise-then-matmul.

TEST INFRASTRUCTURE ONLY (see ``oracle/nvfp4.py``): imported by ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``; never by
the product path.

Stage order and rounding follow the reference's device code
(fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu, cited per function); the
matmuls are plain dense products over dequantised operands, which is what the
reference's own torch check does (fused-moe/test_verdict_moe_ext.py:196-218).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import nvfp4


# --------------------------------------------------------------------------
# a1: router
# --------------------------------------------------------------------------
def route(logits: np.ndarray, topk: int):
    """Softmax over all experts, top-k, renormalise.

    fused-moe/csrc/megakernel_v1.cu:491-537: fp32 softmax with max-subtraction
    (:501-512), insertion of every expert with a strict ``>`` so that the
    **lowest expert id wins a tie** and the result is in descending
    probability order (:515-529), then the selected probabilities are divided
    by their own sum (:531-534).  Sums run sequentially in expert / rank order
    in float32, as the single device thread does.

    Rows with a NaN or +inf logit: in the reference every probability of such a
    row is NaN (``inf - inf``, or a NaN sum), no comparison succeeds and the ids
    stay -1 (:516-528) -- an index nothing downstream can use.  Pinned here
    instead: a NaN probability counts as 0 for the selection, so ids are always
    distinct and in range (``0 .. T-1`` for such a row, lowest id wins the tie)
    and the row's weights come out NaN (``0 / 0``), which marks the token's
    output as invalid without any out-of-range access.

    Returns ``(topk_ids int32 [M, T], topk_weights float32 [M, T])``.
    """
    logits = np.asarray(logits, dtype=np.float32)
    M, E = logits.shape
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        mx = np.fmax.reduce(logits, axis=1, keepdims=True, initial=-np.inf)     # fmaxf skips NaN
        ex = np.exp((logits - mx).astype(np.float32)).astype(np.float32)
        # sequential float32 sum (np.add.accumulate does not pair-wise reduce)
        s = np.add.accumulate(ex, axis=1, dtype=np.float32)[:, -1:]
        p = (ex * (np.float32(1.0) / s)).astype(np.float32)
        p = np.where(np.isnan(p), np.float32(0), p)
        order = np.argsort(-p, axis=1, kind="stable")[:, :topk]
        sel = np.take_along_axis(p, order, axis=1)
        ssum = np.add.accumulate(sel, axis=1, dtype=np.float32)[:, -1:]
        w = (sel * (np.float32(1.0) / ssum)).astype(np.float32)
    return order.astype(np.int32), w


def route_ids_are_unambiguous(logits: np.ndarray, topk: int) -> bool:
    """True when no two probabilities that decide the selection collapse to the
    same float32 value for *different* logits.  When this holds the selected
    ids do not depend on the last-bit behaviour of ``expf`` and must match a
    device implementation exactly."""
    logits = np.asarray(logits, dtype=np.float32)
    mx = np.max(logits, axis=1, keepdims=True)
    p = np.exp((logits - mx).astype(np.float32)).astype(np.float32)
    for m in range(logits.shape[0]):
        o = np.argsort(-p[m], kind="stable")
        head = o[: topk + 1]
        for a, b in zip(head[:-1], head[1:]):
            if p[m, a] == p[m, b] and logits[m, a] != logits[m, b]:
                return False
    return True


# --------------------------------------------------------------------------
# a4: expert-parallel remap
# --------------------------------------------------------------------------
def apply_expert_map(topk_ids: np.ndarray, topk_weights: np.ndarray, expert_map):
    """fused-moe/verdict_moe.py:473-477: ``local = expert_map[ids]``; the weight
    of a pair whose expert is not local (-1) becomes 0 and its id is clamped to
    0, so it contributes exactly nothing."""
    if expert_map is None:
        return topk_ids, topk_weights
    local = np.asarray(expert_map, dtype=np.int32)[topk_ids]
    keep = local != -1
    return np.maximum(local, 0).astype(np.int32), (topk_weights * keep).astype(np.float32)


# --------------------------------------------------------------------------
# a2 / a3: pair tables and the permutation by expert
# --------------------------------------------------------------------------
@dataclass
class GroupTables:
    """Outputs of the stable sort of pairs by expert
    (fused-moe/csrc/verdict_fused_grouped.cu:655-691)."""
    expert_list: np.ndarray          # [G] experts that received at least one pair, ascending
    expert_token_count: np.ndarray   # [G]
    expert_token_offset: np.ndarray  # [G + 1] exclusive prefix sum
    gather_idx: np.ndarray           # [P'] source token of each sorted slot
    scatter_weights: np.ndarray      # [P'] router weight of each sorted slot
    # dense forms (one entry per expert id), as vLLM's expert_offsets / a_map / c_map
    # named in fused-moe/sm120_fused_moe_experts.py:97-107
    expert_offsets: np.ndarray       # [E + 1]
    sorted_pair: np.ndarray          # [P'] flat pair index m*T + j of each sorted slot
    pair_slot: np.ndarray            # [P] sorted slot of each pair, -1 if dropped


def build_group_tables(topk_ids: np.ndarray, topk_weights: np.ndarray, num_experts: int,
                       keep: np.ndarray | None = None) -> GroupTables:
    """Stable sort of the flat pairs (token-major, ``p = m*T + j``, ``token =
    p // T`` as fused-moe/verdict_moe.py:285-291,490-496) by expert id; token
    order is preserved inside an expert.  ``keep`` (bool ``[M, T]``) drops pairs
    (expert-parallel: pairs whose expert lives on another GPU)."""
    ids = np.asarray(topk_ids, dtype=np.int32)
    M, T = ids.shape
    flat = ids.reshape(-1)
    w = np.asarray(topk_weights, dtype=np.float32).reshape(-1)
    pairs = np.arange(M * T, dtype=np.int32)
    if keep is not None:
        pairs = pairs[np.asarray(keep, dtype=bool).reshape(-1)]
    order = pairs[np.argsort(flat[pairs], kind="stable")]
    counts = np.bincount(flat[order], minlength=num_experts).astype(np.int32)
    offsets = np.zeros(num_experts + 1, dtype=np.int32)
    np.cumsum(counts, out=offsets[1:])
    active = np.nonzero(counts)[0].astype(np.int32)
    pair_slot = np.full(M * T, -1, dtype=np.int32)
    pair_slot[order] = np.arange(order.size, dtype=np.int32)
    act_off = np.zeros(active.size + 1, dtype=np.int32)
    np.cumsum(counts[active], out=act_off[1:])
    return GroupTables(
        expert_list=active,
        expert_token_count=counts[active],
        expert_token_offset=act_off,
        gather_idx=(order // T).astype(np.int32),
        scatter_weights=w[order],
        expert_offsets=offsets,
        sorted_pair=order.astype(np.int32),
        pair_slot=pair_slot,
    )


# --------------------------------------------------------------------------
# a6 .. a12: the layer
# --------------------------------------------------------------------------
def silu(x: np.ndarray) -> np.ndarray:
    """``x / (1 + expf(-x))`` in float32
    (fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:64-66)."""
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (x / (np.float32(1.0) + np.exp(-x).astype(np.float32))).astype(np.float32)


def _matmul_t(a: np.ndarray, w: np.ndarray, accum: str) -> np.ndarray:
    """``a [m, K] @ w[n, K].T`` -> float32."""
    if accum == "f64":
        return (a.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    import torch  # multi-threaded sgemm; the reference's check uses torch too
    return (torch.from_numpy(a) @ torch.from_numpy(w).T).numpy()


@dataclass
class ExpertWeights:
    """NVFP4 expert weights in the reference's layout
    (fused-moe/verdict_moe.py:571-575,519-520): ``w13 [E, 2N, K/2]`` with rows
    0..N-1 = gate and N..2N-1 = up, ``w13_sf [E, 2N, K/16]`` linear E4M3 bytes,
    ``w2 [E, K, N/2]``, ``w2_sf [E, K, N/16]``; ``*_gs [E]`` float32 global
    scales (``weight_scale_2``), which play the part of the reference's
    ``alpha`` (fused-moe/verdict_moe.py:499-513)."""
    w13: np.ndarray
    w13_sf: np.ndarray
    w13_gs: np.ndarray
    w2: np.ndarray
    w2_sf: np.ndarray
    w2_gs: np.ndarray

    @property
    def num_experts(self):
        return self.w13.shape[0]

    @property
    def hidden(self):
        return self.w13.shape[2] * 2

    @property
    def inter(self):
        return self.w2.shape[2] * 2


def expert_mlp(x_packed, x_sf, ew: ExpertWeights, e: int, accum: str = "f64",
               return_inter: bool = False, requant: dict | None = None):
    """One expert on already-quantised token rows: GEMM1 -> x alpha1 -> SwiGLU ->
    requantise -> GEMM2.  Returns the float32 GEMM2 sums ``[m, K]``; the caller
    multiplies them by ``router_weight * alpha2``.

    Stage order: fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu
    :323-400 (GEMM1, fp32 accumulate of ``a_q sa w_q sw``), :426-428 (``gate
    *= alpha1; up *= alpha1; s = up * silu(gate)``), :430-452 (requantise per
    16 consecutive n, no global scale on the intermediate), :460-527 (GEMM2).
    """
    N = ew.inter
    a = nvfp4.dequantize(x_packed, x_sf)                       # [m, K]
    w1 = nvfp4.dequantize(ew.w13[e], ew.w13_sf[e])             # [2N, K], block scales only
    acc = _matmul_t(a, w1, accum)                              # [m, 2N]
    alpha1 = np.float32(ew.w13_gs[e])
    gate = (acc[:, :N] * alpha1).astype(np.float32)
    up = (acc[:, N:] * alpha1).astype(np.float32)
    s = (up * silu(gate)).astype(np.float32)
    # requant: options of the intermediate quantiser (default: the device rules); the host harness of the
    # reference uses tie="low", scale_round="ceil" (fused-moe/csrc/verdict_fused_independent.cu:474-496)
    s_packed, s_sf = nvfp4.quantize_act(s, **(requant or {}))
    sq = nvfp4.dequantize(s_packed, s_sf)                      # [m, N]
    w2 = nvfp4.dequantize(ew.w2[e], ew.w2_sf[e])               # [K, N]
    y = _matmul_t(sq, w2, accum)                               # [m, K], alpha2 not applied
    if return_inter:
        return y, s_packed, s_sf, s
    return y


def moe_layer(hidden_bf16: np.ndarray, topk_ids: np.ndarray, topk_weights: np.ndarray,
              ew: ExpertWeights, shared: ExpertWeights | None = None,
              expert_map=None, accum: str = "f64", return_stages: bool = False):
    """The fused NVFP4 MoE expert layer.

    ``hidden_bf16`` is float32 holding bf16-representable values ``[M, K]``.
    a6: quantise every token once (…tma_ext.cu:249-279); a8-a10 per pair;
    a10: ``pair_out = (router_weight * alpha2) * y`` (:529-537, the product of
    the two scalars is formed first); a11: ``out = bf16(sum over the token's
    pairs in ascending pair order)`` in float32 (:549-563); a12: the always-on
    shared expert is one more pair with router weight 1.0
    (fused-moe/csrc/megakernel_v1.cu:1431-1505), added after the routed pairs.
    """
    x = np.asarray(hidden_bf16, dtype=np.float32)
    M, K = x.shape
    T = topk_ids.shape[1]
    ids, wts = apply_expert_map(np.asarray(topk_ids, np.int32),
                                np.asarray(topk_weights, np.float32), expert_map)
    xq, xsf = nvfp4.quantize_act(x)
    pair_out = np.zeros((M, T + (1 if shared is not None else 0), K), dtype=np.float32)
    inter = {}
    # visit each distinct expert once, all of its tokens together
    live = wts != 0 if expert_map is not None else np.ones_like(ids, dtype=bool)
    for e in np.unique(ids[live]):
        toks, js = np.nonzero((ids == e) & live)
        res = expert_mlp(xq[toks], xsf[toks], ew, int(e), accum, return_inter=return_stages)
        y = res[0] if return_stages else res
        scale = (wts[toks, js] * np.float32(ew.w2_gs[e])).astype(np.float32)
        pair_out[toks, js] = (y * scale[:, None]).astype(np.float32)
        if return_stages:
            for k, (t, j) in enumerate(zip(toks, js)):
                inter[(int(t), int(j))] = (res[1][k], res[2][k], res[3][k])
    if shared is not None:
        res = expert_mlp(xq, xsf, shared, 0, accum, return_inter=return_stages)
        y = res[0] if return_stages else res
        pair_out[:, T] = (y * (np.float32(1.0) * np.float32(shared.w2_gs[0]))).astype(np.float32)
        if return_stages:
            for t in range(M):
                inter[(t, T)] = (res[1][t], res[2][t], res[3][t])
    acc = np.zeros((M, K), dtype=np.float32)
    for j in range(pair_out.shape[1]):                      # fixed ascending order, float32
        acc = (acc + pair_out[:, j]).astype(np.float32)
    out = nvfp4.bf16_round(acc)
    if return_stages:
        return out, dict(xq=xq, xsf=xsf, pair_out=pair_out, inter=inter, acc=acc)
    return out


def moe_layer_from_logits(hidden_bf16, logits, topk, ew, shared=None, expert_map=None,
                          accum="f64"):
    ids, w = route(logits, topk)
    return moe_layer(hidden_bf16, ids, w, ew, shared, expert_map, accum)


# --------------------------------------------------------------------------
# behind the layer: RMSNorm + activation quantisation of the next layer's input
# --------------------------------------------------------------------------
def rmsnorm_quantize(x_bf16: np.ndarray, gamma: np.ndarray, eps: float = 1e-6, threads: int = 256):
    """RMSNorm of bf16 rows and NVFP4 quantisation of the result, as the next layer's GEMM wants it.

    fused-moe/csrc/megakernel_v1.cu:257-352 (``rmsnorm_parallel`` + ``rmsnorm_apply_and_quantize``): sum of
    squares over the row, ``rms = 1 / sqrt(sum / K + eps)``, ``norm = x * rms * weight``, then the per-16 block
    quantiser.  The reference holds the row in float32 and sums with atomics (order undefined); pinned here: the
    row is bf16, the sum of squares runs in the device's fixed order -- ``threads`` partial sums, thread ``t`` over
    the 16-element blocks ``t, t + threads, ...`` in element order; a 32-wide xor tree (16, 8, 4, 2, 1) inside
    each warp; then the warp sums in warp order -- the reciprocal square root is exact IEEE arithmetic, and the
    normalised row is rounded to bf16 before it is quantised.

    Returns ``(y float32 holding bf16 values [M, K], packed u8 [M, K/2], sf u8 [M, K/16])``.
    """
    x = np.asarray(x_bf16, dtype=np.float32)
    g = np.asarray(gamma, dtype=np.float32)
    M, K = x.shape
    nblk = K // 16
    sq = (x * x).astype(np.float32)                       # exact: bf16 x bf16 fits float32
    part = np.zeros((M, threads), np.float32)
    blocks = sq.reshape(M, nblk, 16)
    for b0 in range(0, nblk, threads):                    # every thread walks its blocks in order
        chunk = blocks[:, b0:b0 + threads]                # [M, <=threads, 16]
        for i in range(16):
            part[:, :chunk.shape[1]] = (part[:, :chunk.shape[1]] + chunk[:, :, i]).astype(np.float32)
    lanes = np.arange(32)
    w = part.reshape(M, threads // 32, 32)
    for o in (16, 8, 4, 2, 1):
        w = (w + w[:, :, lanes ^ o]).astype(np.float32)
    total = np.zeros(M, np.float32)
    for k in range(threads // 32):
        total = (total + w[:, k, 0]).astype(np.float32)
    mean = (total / np.float32(K)).astype(np.float32)
    rms = (np.float32(1.0) / np.sqrt((mean + np.float32(eps)).astype(np.float32)).astype(np.float32)).astype(np.float32)
    y = nvfp4.bf16_round(((x * rms[:, None]).astype(np.float32) * g[None, :]).astype(np.float32))
    packed, sf = nvfp4.quantize_act(y)
    return y, packed, sf
