"""Checkpoint ingestion: per-expert NVFP4 tensors of a safetensors checkpoint -> the stacked layout of the
operator (``w13 [E, 2N, K/2]``, ``w13_sf [E, 2N, K/16]``, ``w13_gs [E]``, ``w2 [E, K, N/2]``,
``w2_sf [E, K, N/16]``, ``w2_gs [E]``).

Follows the reference's loader (fused-moe/ep_moe_poc.py:26-57: ``<prefix>.{gate,up,down}_proj.{weight,
weight_scale,weight_scale_2}`` per expert, uint8 codes, float8_e4m3fn block scales, fp32 global scale) and
its stacking (``w1 = cat([gate, up])``, :217-228).  The gate and up projections of an expert share ONE
global scale in the stacked form (as vLLM's ``w13_weight_scale_2``); a checkpoint whose two scales differ is
refused unless ``allow_scale_mismatch`` is set, in which case the gate scale is used for both, as vLLM does.
"""
from __future__ import annotations

import glob
import json
import os

import torch

DEFAULT_EXPERT_PREFIX = "model.language_model.layers.{layer}.mlp.experts.{expert}"
DEFAULT_SHARED_PREFIX = "model.language_model.layers.{layer}.mlp.shared_expert"
_PROJ = ("gate_proj", "up_proj", "down_proj")
_PARTS = ("weight", "weight_scale", "weight_scale_2")


class _Shards:
    """Tensor name -> file, from ``model.safetensors.index.json`` when present, else by opening every shard."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        self._open = safe_open
        self.dir = model_dir
        self.where: dict[str, str] = {}
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
                with safe_open(path, framework="pt", device="cpu") as f:
                    for k in f.keys():
                        self.where[k] = os.path.basename(path)
        if not self.where:
            raise FileNotFoundError(f"no safetensors tensors under {model_dir}")
        self._handles: dict[str, object] = {}

    def get(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise KeyError(f"tensor {name!r} is not in the checkpoint")
        fn = self.where[name]
        if fn not in self._handles:
            self._handles[fn] = self._open(os.path.join(self.dir, fn), framework="pt", device="cpu")
        return self._handles[fn].get_tensor(name)


def _as_u8(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.uint8:
        return t
    if t.dtype in (torch.float8_e4m3fn, torch.int8):
        return t.view(torch.uint8)
    raise TypeError(f"expected uint8 / float8_e4m3fn bytes, got {t.dtype}")


def _one_expert(sh: _Shards, prefix: str, allow_scale_mismatch: bool):
    t = {(p, q): sh.get(f"{prefix}.{p}.{q}") for p in _PROJ for q in _PARTS}
    gate_w, up_w, down_w = (_as_u8(t[(p, "weight")]) for p in _PROJ)
    gate_s, up_s, down_s = (_as_u8(t[(p, "weight_scale")]) for p in _PROJ)
    gate_g, up_g, down_g = (t[(p, "weight_scale_2")].float().reshape(-1) for p in _PROJ)
    n, k2 = gate_w.shape
    if up_w.shape != (n, k2) or down_w.shape != (2 * k2, n // 2):
        raise ValueError(f"{prefix}: shapes gate {tuple(gate_w.shape)}, up {tuple(up_w.shape)}, down {tuple(down_w.shape)} "
                         "are not [N, K/2], [N, K/2], [K, N/2]")
    if gate_s.shape != (n, k2 // 8) or up_s.shape != (n, k2 // 8) or down_s.shape != (2 * k2, n // 16):
        raise ValueError(f"{prefix}: block scales are not one per 16 elements")
    if not torch.equal(gate_g, up_g) and not allow_scale_mismatch:
        raise ValueError(f"{prefix}: gate_proj and up_proj have different global scales "
                         f"({gate_g.item()} vs {up_g.item()}); the stacked layout holds one")
    return (torch.cat([gate_w, up_w], 0), torch.cat([gate_s, up_s], 0), gate_g[0],
            down_w, down_s, down_g[0])


def load_moe_layer(model_dir: str, layer: int, num_experts: int, *, expert_prefix: str = DEFAULT_EXPERT_PREFIX,
                   shared_prefix: str | None = None, first_expert: int = 0, device="cpu",
                   allow_scale_mismatch: bool = False):
    """Returns ``dict(routed=6-tuple, shared=6-tuple or None)`` in the argument order of ``ops.MoEWeights``.
    ``first_expert`` / ``num_experts`` select a contiguous block (one rank's share under expert parallelism)."""
    sh = _Shards(model_dir)
    per = [_one_expert(sh, expert_prefix.format(layer=layer, expert=first_expert + e), allow_scale_mismatch)
           for e in range(num_experts)]

    def stack(items):
        w13 = torch.stack([i[0] for i in items]).contiguous()
        w13_sf = torch.stack([i[1] for i in items]).contiguous()
        w13_gs = torch.stack([i[2] for i in items]).float().contiguous()
        w2 = torch.stack([i[3] for i in items]).contiguous()
        w2_sf = torch.stack([i[4] for i in items]).contiguous()
        w2_gs = torch.stack([i[5] for i in items]).float().contiguous()
        return tuple(t.to(device) for t in (w13, w13_sf, w13_gs, w2, w2_sf, w2_gs))

    out = dict(routed=stack(per), shared=None)
    if shared_prefix is not None:
        out["shared"] = stack([_one_expert(sh, shared_prefix.format(layer=layer), allow_scale_mismatch)])
    return out


def save_moe_layer(model_dir: str, layer: int, routed, shared=None, *, expert_prefix: str = DEFAULT_EXPERT_PREFIX,
                   shared_prefix: str = DEFAULT_SHARED_PREFIX, shards: int = 2) -> None:
    """Inverse of ``load_moe_layer`` (synthetic checkpoints for tests and benchmarks): writes the stacked tensors
    as per-expert ``gate_proj / up_proj / down_proj`` entries over ``shards`` files plus the index file."""
    from safetensors.torch import save_file
    os.makedirs(model_dir, exist_ok=True)

    def split(prefix, w13, w13_sf, w13_gs, w2, w2_sf, w2_gs):
        n = w13.shape[0] // 2
        return {
            f"{prefix}.gate_proj.weight": w13[:n].contiguous(), f"{prefix}.up_proj.weight": w13[n:].contiguous(),
            f"{prefix}.gate_proj.weight_scale": w13_sf[:n].contiguous().view(torch.float8_e4m3fn),
            f"{prefix}.up_proj.weight_scale": w13_sf[n:].contiguous().view(torch.float8_e4m3fn),
            f"{prefix}.gate_proj.weight_scale_2": w13_gs.reshape(1).clone(), f"{prefix}.up_proj.weight_scale_2": w13_gs.reshape(1).clone(),
            f"{prefix}.down_proj.weight": w2.contiguous(), f"{prefix}.down_proj.weight_scale": w2_sf.contiguous().view(torch.float8_e4m3fn),
            f"{prefix}.down_proj.weight_scale_2": w2_gs.reshape(1).clone(),
        }

    files: list[dict] = [dict() for _ in range(shards)]
    E = routed[0].shape[0]
    for e in range(E):
        files[e % shards].update(split(expert_prefix.format(layer=layer, expert=e), *[t[e].cpu() for t in routed]))
    if shared is not None:
        files[0].update(split(shared_prefix.format(layer=layer), *[t[0].cpu() for t in shared]))
    weight_map = {}
    for i, tensors in enumerate(files):
        name = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        save_file(tensors, os.path.join(model_dir, name))
        weight_map.update({k: name for k in tensors})
    with open(os.path.join(model_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
