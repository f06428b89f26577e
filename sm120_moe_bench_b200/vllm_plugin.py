"""Runtime registration of ``VerdictMoEExperts`` as an NVFP4 MoE backend of vLLM.

The reference edits vLLM's installed ``oracle/nvfp4.py`` as text (fused-moe/patches/
nvfp4_oracle_verdict.py:21-83): it adds a ``VERDICT_MOE`` member to ``NvFp4MoeBackend``, maps it to
``[VerdictMoEExperts]`` in ``backend_to_kernel_cls``, selects it when ``VLLM_USE_VERDICT_MOE=1`` and adds
``"verdict_moe"`` to ``map_nvfp4_backend``; and it copies the operator into the vLLM package (:86-104).
``install()`` does the same in memory, without touching a file of vLLM: the oracle's functions are
wrapped and every module that already imported them by name is re-pointed at the wrappers.  It can be
called by hand before the engine is built or listed as a ``vllm.general_plugins`` entry point.

What the backend asks of the framework (the reference's PHASE2 notes, fused-moe/PHASE2_RESULTS.md:26-28):
weights and block scales stay in checkpoint layout (linear ``[E, rows, K/16]`` scales, not swizzled),
``g1_alphas / g2_alphas`` are the raw per-expert weight global scales, activations are quantised inside
the kernels per 16-element block without a global scale.  The 128-row scale atoms the tcgen05 kernels
read are produced once, by ``process_weights_after_loading`` -> ``MoEWeights.prepare()``.
"""
from __future__ import annotations

import os
import sys

ENV_FLAG = "VLLM_USE_VERDICT_MOE"          # same switch as the reference's patch
BACKEND_NAME = "verdict_moe"               # value for ``moe_backend=``

_ORACLE = "vllm.model_executor.layers.fused_moe.oracle.nvfp4"
_WRAPPED = ("backend_to_kernel_cls", "map_nvfp4_backend", "select_nvfp4_moe_backend",
            "convert_to_nvfp4_moe_kernel_format", "make_nvfp4_moe_quant_config",
            "is_global_sf_supported_for_nvfp4_backend")
_originals: dict = {}


class _VerdictBackend:
    """Stands in for the enum member the reference adds: compares equal only to itself, has ``.value``."""
    value = "VERDICT_MOE"
    name = "VERDICT_MOE"

    def __repr__(self):
        return "<NvFp4MoeBackend.VERDICT_MOE: 'VERDICT_MOE'>"


VERDICT_MOE = _VerdictBackend()


def _kernel_classes():
    from .verdict_moe import VerdictMoEExperts
    return [VerdictMoEExperts]


def _wants_verdict(config) -> bool:
    if os.environ.get(ENV_FLAG, "0") == "1":
        return True
    return getattr(config, "moe_backend", "auto") == BACKEND_NAME


def _make_wrappers(oracle):
    import vllm.model_executor.layers.fused_moe.modular_kernel as mk
    from vllm.model_executor.layers.fused_moe.config import nvfp4_moe_quant_config

    o = {n: getattr(oracle, n) for n in _WRAPPED}

    def backend_to_kernel_cls(backend):
        if backend is VERDICT_MOE:
            return _kernel_classes()
        return o["backend_to_kernel_cls"](backend)

    def map_nvfp4_backend(runner_backend):
        if runner_backend == BACKEND_NAME:
            return VERDICT_MOE
        return o["map_nvfp4_backend"](runner_backend)

    def select_nvfp4_moe_backend(config, weight_key, activation_key):
        if not _wants_verdict(config):
            return o["select_nvfp4_moe_backend"](config, weight_key, activation_key)
        use_batched = config.moe_parallel_config.use_batched_activation_format
        fmt = (mk.FusedMoEActivationFormat.BatchedExperts if use_batched
               else mk.FusedMoEActivationFormat.Standard)
        reason = None
        for k_cls in _kernel_classes():
            ok, reason = k_cls.is_supported_config(k_cls, config, weight_key, activation_key, fmt)
            if ok:
                return VERDICT_MOE, k_cls
        # asked for explicitly: fail loudly, as the oracle does for an explicit backend (no silent fallback)
        raise ValueError(f"NvFp4 MoE backend 'VERDICT_MOE' does not support the deployment configuration"
                         f"{' since ' + reason if reason else ''}.")

    def convert_to_nvfp4_moe_kernel_format(nvfp4_backend, layer, w13, w13_scale, w13_scale_2, a13_scale,
                                           w2, w2_scale, w2_scale_2, a2_scale, is_act_and_mul):
        if nvfp4_backend is VERDICT_MOE:
            # checkpoint layout is the kernel layout: nothing is swizzled, padded or reordered here
            return w13, w13_scale, w13_scale_2, a13_scale, w2, w2_scale, w2_scale_2, a2_scale
        return o["convert_to_nvfp4_moe_kernel_format"](nvfp4_backend, layer, w13, w13_scale, w13_scale_2, a13_scale,
                                                       w2, w2_scale, w2_scale_2, a2_scale, is_act_and_mul)

    def make_nvfp4_moe_quant_config(backend, w13_scale, w2_scale, w13_scale_2, w2_scale_2, a13_scale, a2_scale,
                                    swiglu_limit=None):
        if backend is VERDICT_MOE:
            if swiglu_limit is not None:
                raise ValueError("VERDICT_MOE does not apply a SwiGLU clamp")
            return nvfp4_moe_quant_config(g1_alphas=w13_scale_2, g2_alphas=w2_scale_2,
                                          a1_gscale=(1.0 / a13_scale), a2_gscale=(1.0 / a2_scale),
                                          w1_scale=w13_scale, w2_scale=w2_scale, is_scale_swizzled=False)
        return o["make_nvfp4_moe_quant_config"](backend, w13_scale, w2_scale, w13_scale_2, w2_scale_2, a13_scale,
                                                a2_scale, swiglu_limit)

    def is_global_sf_supported_for_nvfp4_backend(backend):
        if backend is VERDICT_MOE:
            return False
        return o["is_global_sf_supported_for_nvfp4_backend"](backend)

    return o, {"backend_to_kernel_cls": backend_to_kernel_cls, "map_nvfp4_backend": map_nvfp4_backend,
               "select_nvfp4_moe_backend": select_nvfp4_moe_backend,
               "convert_to_nvfp4_moe_kernel_format": convert_to_nvfp4_moe_kernel_format,
               "make_nvfp4_moe_quant_config": make_nvfp4_moe_quant_config,
               "is_global_sf_supported_for_nvfp4_backend": is_global_sf_supported_for_nvfp4_backend}


def install() -> bool:
    """Register the backend.  Returns False when vLLM (or its NVFP4 oracle) is not importable, True otherwise.
    Idempotent.  The operator then reads the raw weight global scales (``alpha_convention = "weight"``)."""
    global _originals
    if _originals:
        return True
    try:
        import importlib
        oracle = importlib.import_module(_ORACLE)
    except Exception:  # noqa: BLE001 - vLLM absent or a different layout: nothing to register
        return False
    if not all(hasattr(oracle, n) for n in _WRAPPED):
        return False
    originals, wrappers = _make_wrappers(oracle)
    # the oracle module itself, then every module that did ``from ...oracle.nvfp4 import <name>``
    for mod in list(sys.modules.values()):
        if mod is None or not getattr(mod, "__name__", "").startswith("vllm"):
            continue
        for name, orig in originals.items():
            try:
                if getattr(mod, name, None) is orig:
                    setattr(mod, name, wrappers[name])
            except Exception:  # noqa: BLE001 - read-only module objects
                pass
    _originals = originals
    from . import verdict_moe
    verdict_moe._VerdictCommon.alpha_convention = os.environ.get("VMOE_ALPHA_CONVENTION", "weight")
    return True


def uninstall() -> None:
    """Put the oracle's own functions back (tests)."""
    global _originals
    if not _originals:
        return
    import importlib
    oracle = importlib.import_module(_ORACLE)
    current = {n: getattr(oracle, n) for n in _WRAPPED}
    for mod in list(sys.modules.values()):
        if mod is None or not getattr(mod, "__name__", "").startswith("vllm"):
            continue
        for name, orig in _originals.items():
            try:
                if getattr(mod, name, None) is current[name]:
                    setattr(mod, name, orig)
            except Exception:  # noqa: BLE001
                pass
    _originals = {}


def register() -> None:
    """Entry point for ``vllm.general_plugins``."""
    install()
