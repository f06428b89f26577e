"""Child process of tests/test_abi_cpu.py: registers the backend with the installed vLLM (no GPU needed) and
checks the four changes of fused-moe/patches/nvfp4_oracle_verdict.py: backend -> class, name -> backend,
VLLM_USE_VERDICT_MOE=1 selection, plus un-swizzled scales and raw weight global scales in the quant config."""
import os
import sys
import types

import torch

os.environ["VMOE_NO_VLLM"] = "0"
try:
    import vllm.model_executor.layers.fused_moe.oracle.nvfp4 as oracle
except Exception:  # noqa: BLE001
    print("NOVLLM")
    raise SystemExit(0)

from sm120_moe_bench_b200 import verdict_moe as vmo
from sm120_moe_bench_b200 import vllm_plugin as vp

assert vmo.HAVE_VLLM
before = oracle.select_nvfp4_moe_backend
assert vp.install() and vp.install()                     # idempotent
assert oracle.select_nvfp4_moe_backend is not before
assert oracle.backend_to_kernel_cls(vp.VERDICT_MOE) == [vmo.VerdictMoEExperts]
assert oracle.map_nvfp4_backend("verdict_moe") is vp.VERDICT_MOE
assert oracle.map_nvfp4_backend("marlin") is oracle.NvFp4MoeBackend.MARLIN          # others untouched
assert len(oracle.backend_to_kernel_cls(oracle.NvFp4MoeBackend.MARLIN)) == 1
assert oracle.is_global_sf_supported_for_nvfp4_backend(vp.VERDICT_MOE) is False
# modules that imported the functions by name before install() see the wrappers too
for mod in list(sys.modules.values()):
    if mod is not None and getattr(mod, "__name__", "").startswith("vllm") and hasattr(mod, "select_nvfp4_moe_backend"):
        assert mod.select_nvfp4_moe_backend is oracle.select_nvfp4_moe_backend, mod.__name__

# weights keep the checkpoint layout
t = [torch.zeros(1) for _ in range(8)]
out = oracle.convert_to_nvfp4_moe_kernel_format(vp.VERDICT_MOE, None, t[0], t[1], t[2], t[3], t[4], t[5], t[6], t[7], True)
assert all(a is b for a, b in zip(out, t))

# quant config: raw weight global scales, linear (not swizzled) block scales
qc = oracle.make_nvfp4_moe_quant_config(vp.VERDICT_MOE, torch.ones(2, 4, 4), torch.ones(2, 4, 4),
                                        torch.full((2,), 3.0), torch.full((2,), 5.0),
                                        torch.full((2,), 2.0), torch.full((2,), 4.0))
assert torch.equal(qc.g1_alphas, torch.full((2,), 3.0)) and torch.equal(qc.a1_gscale, torch.full((2,), 0.5))
assert qc.is_scale_swizzled is False
assert vmo.VerdictMoEExperts.alpha_convention == "weight"

# selection by the environment switch of the reference; the capability probe is faked (no GPU here)
os.environ[vp.ENV_FLAG] = "1"
seen = {}


def supported(cls, cfg, wk, ak, fmt):
    seen["cls"] = cls
    return True, None


orig_supported = vmo.VerdictMoEExperts.is_supported_config
vmo.VerdictMoEExperts.is_supported_config = staticmethod(supported)
cfg = types.SimpleNamespace(moe_backend="auto",
                            moe_parallel_config=types.SimpleNamespace(use_batched_activation_format=False))
backend, cls = oracle.select_nvfp4_moe_backend(cfg, vmo.kNvfp4Static, vmo.kNvfp4Dynamic)
assert backend is vp.VERDICT_MOE and cls is vmo.VerdictMoEExperts and seen["cls"] is cls
# an unsupported configuration fails loudly instead of falling back to another backend
vmo.VerdictMoEExperts.is_supported_config = staticmethod(lambda cls, cfg, wk, ak, fmt: (False, "kernel does not support it"))
try:
    oracle.select_nvfp4_moe_backend(cfg, vmo.kNvfp4Static, vmo.kNvfp4Dynamic)
    raise SystemExit("expected ValueError")
except ValueError:
    pass
vmo.VerdictMoEExperts.is_supported_config = orig_supported
del os.environ[vp.ENV_FLAG]

# the real probe chain on this host: everything but the device check passes for a standard configuration
assert vmo.VerdictMoEExperts._supports_quant_scheme(vmo.kNvfp4Static, vmo.kNvfp4Dynamic)
assert not vmo.VerdictMoEExperts._supports_no_act_and_mul()

vp.uninstall()
assert oracle.select_nvfp4_moe_backend is before
print("OK")
