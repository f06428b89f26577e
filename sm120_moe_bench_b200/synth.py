"""Seeded synthetic NVFP4 MoE layers (weights, activations, router logits).

They stand in for the checkpoint the reference measured on (Qwen3.5-397B-A17B-NVFP4, not
available offline).  Shapes and value distributions: weights fp32 N(0, 0.02) quantised to NVFP4
with one fp32 global scale per expert per stacked matrix (``gs = amax / (448 * 6)``, so block
scales use the top of the E4M3 range as real checkpoints do), activations bf16 N(0, 1), router
logits fp32 N(0, 1), optionally with a Zipf(s) bias over a seeded permutation of expert ids.

Everything is plain torch and runs on CPU or GPU; the tensor layout is the reference's
(fused-moe/verdict_moe.py:571-575): ``w13 [E, 2N, K/2]``, ``w13_sf [E, 2N, K/16]``,
``w2 [E, K, N/2]``, ``w2_sf [E, K, N/16]``, low nibble = even k.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

E2M1_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


@dataclass(frozen=True)
class LayerConfig:
    name: str
    hidden: int
    inter: int
    num_experts: int
    topk: int
    shared: bool


# BASELINE configs: [0] the tiny CPU-runnable layer, [1..4] the large-MoE shape
CONFIG_TINY = LayerConfig("tiny", 1024, 512, 8, 2, False)
CONFIG_LARGE = LayerConfig("large", 4096, 1024, 512, 10, True)


def quantize_weight(w: torch.Tensor):
    """fp32 ``[E, R, K]`` -> (packed u8 ``[E, R, K/2]``, sf u8 ``[E, R, K/16]``, gs f32 ``[E]``).

    ``value = e2m1(code) * e4m3(sf) * gs`` is the dequantisation the reference applies to
    checkpoint tensors (fused-moe/ep_moe_poc.py:60-98); this is its inverse with the device's
    rounding rules (E4M3 scale: round-to-nearest-even saturating at 448; E2M1 code: thresholds
    compared with ``<``, fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:57-76)."""
    E, R, K = w.shape
    w = w.float()
    gs = (w.abs().amax(dim=(1, 2)).clamp_min(1e-30) / (448.0 * 6.0)).float()
    blocks = w.view(E, R, K // 16, 16)
    bmax = blocks.abs().amax(dim=-1)
    target = (bmax / (6.0 * gs).view(E, 1, 1)).clamp(max=448.0)
    sf = target.to(torch.float8_e4m3fn)
    scale = sf.float().clamp_min(1e-30) * gs.view(E, 1, 1)
    scaled = blocks / scale.unsqueeze(-1)
    av = scaled.abs()
    idx = torch.zeros_like(av, dtype=torch.uint8)
    for t in E2M1_THRESHOLDS:
        idx += (~(av < t)).to(torch.uint8)
    codes = (idx | ((scaled < 0).to(torch.uint8) << 3)).view(E, R, K)
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)
    return packed.contiguous(), sf.view(torch.uint8).contiguous(), gs.contiguous()


def make_expert_weights(num_experts: int, hidden: int, inter: int, generator: torch.Generator,
                        device="cpu", std: float = 0.02, chunk: int = 16):
    """``(w13, w13_sf, w13_gs, w2, w2_sf, w2_gs)`` drawn expert-chunk by expert-chunk."""
    outs = [[] for _ in range(6)]
    for e0 in range(0, num_experts, chunk):
        n = min(chunk, num_experts - e0)
        w13 = torch.randn(n, 2 * inter, hidden, generator=generator, device=device) * std
        p, s, g = quantize_weight(w13)
        del w13
        outs[0].append(p); outs[1].append(s); outs[2].append(g)
        w2 = torch.randn(n, hidden, inter, generator=generator, device=device) * std
        p, s, g = quantize_weight(w2)
        del w2
        outs[3].append(p); outs[4].append(s); outs[5].append(g)
    return tuple(torch.cat(o) for o in outs)


def make_layer(cfg: LayerConfig, seed: int = 0, device="cpu"):
    """Returns ``dict(routed=6-tuple, shared=6-tuple or None)`` of tensors on ``device``.
    On CPU the draw comes from ``torch.manual_seed``-style CPU generator (bit-reproducible
    anywhere); on GPU from a CUDA generator with the same seed (reproducible per GPU model)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    routed = make_expert_weights(cfg.num_experts, cfg.hidden, cfg.inter, gen, device)
    shared = make_expert_weights(1, cfg.hidden, cfg.inter, gen, device) if cfg.shared else None
    return dict(routed=routed, shared=shared)


def make_inputs(cfg: LayerConfig, tokens: int, seed: int = 0, device="cpu", zipf_s: float | None = None,
                mtp_group: int | None = None, mtp_corr: float = 0.0):
    """bf16 activations N(0,1) ``[M, K]`` and fp32 router logits N(0,1) ``[M, E]``; with
    ``zipf_s`` the bias ``log(rank ** -s)`` over a seeded permutation of expert ids is added.

    ``mtp_group`` / ``mtp_corr``: consecutive groups of ``mtp_group`` tokens stand for the positions of one
    sequence under multi-token prediction (1 verified + 5 speculative draft positions at 6).  Their logits share a
    seeded component, ``l_i = c * base + sqrt(1 - c^2) * own_i`` (still N(0,1) each), so adjacent positions reuse
    part of their experts, as the reference observed on real traffic (71 % adjacent-token expert reuse,
    RELEASE_MANIFEST.md:108-110); ``c = 0.98`` gives about that figure for 512 experts, top-10."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 1000003)
    hidden = torch.randn(tokens, cfg.hidden, generator=gen, device=device).to(torch.bfloat16)
    logits = torch.randn(tokens, cfg.num_experts, generator=gen, device=device)
    if mtp_group and mtp_corr > 0.0:
        if tokens % mtp_group:
            raise ValueError("tokens must be a multiple of mtp_group")
        base = torch.randn(tokens // mtp_group, 1, cfg.num_experts, generator=gen, device=device)
        own = logits.view(tokens // mtp_group, mtp_group, cfg.num_experts)
        logits = (mtp_corr * base + (1.0 - mtp_corr * mtp_corr) ** 0.5 * own).reshape(tokens, cfg.num_experts)
    if zipf_s is not None:
        perm = torch.randperm(cfg.num_experts, generator=gen, device=device)
        rank = torch.empty(cfg.num_experts, device=device)
        rank[perm] = torch.arange(1, cfg.num_experts + 1, device=device, dtype=torch.float32)
        logits = logits + (-zipf_s) * torch.log(rank)
    return hidden, logits.float().contiguous()


def adjacent_reuse(topk_ids: torch.Tensor, group: int) -> float:
    """Fraction of a position's experts that the next position of the same sequence also selected."""
    M, T = topk_ids.shape
    sel = torch.zeros(M, int(topk_ids.max()) + 1, dtype=torch.bool, device=topk_ids.device)
    sel.scatter_(1, topk_ids.long(), True)
    sel = sel.view(M // group, group, -1)
    return float((sel[:, 1:] & sel[:, :-1]).sum(-1).float().mean() / T)
