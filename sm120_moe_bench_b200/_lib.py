"""ctypes binding of ``libvmoe.so`` (the C ABI declared in ``include/vmoe.h``).

There is no fallback: if the library is missing or a symbol cannot be resolved the import of
this module raises, and every operator in the package fails with it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libvmoe.so"


class VmoeShape(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("num_experts", C.c_int32),
                ("topk", C.c_int32), ("max_tokens", C.c_int32), ("has_shared", C.c_int32),
                ("num_global_experts", C.c_int32), ("path", C.c_int32)]


class VmoeWeights(C.Structure):
    _fields_ = [("w13", C.c_void_p), ("w13_sf", C.c_void_p), ("w13_gs", C.c_void_p),
                ("w2", C.c_void_p), ("w2_sf", C.c_void_p), ("w2_gs", C.c_void_p),
                ("w13_sf_atoms", C.c_void_p), ("w2_sf_atoms", C.c_void_p)]


_LAYOUT_FIELDS = ["total_bytes", "topk_ids", "topk_weights", "expert_offsets", "sorted_pair",
                  "pair_slot", "gather_idx", "scatter_weights", "units", "counters", "act_q",
                  "act_sf", "inter_q", "inter_sf", "pair_out", "bitmap", "word_prefix", "tc_units",
                  "tc_unit_base", "act_q_sorted", "act_sf_atoms", "inter_sf_atoms", "unit_done", "token_done",
                  "token_expect"]


class VmoeEpCtx(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("experts_per_rank", C.c_int32),
                ("capacity", C.c_int32), ("max_local_tokens", C.c_int32), ("wait_limit_us", C.c_int32),
                ("reserved", C.c_int32 * 2),
                ("slab", C.c_void_p * 16)]


class VmoeWsLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in _LAYOUT_FIELDS]


class VmoeExtras(C.Structure):
    _fields_ = [("gate_weight", C.c_void_p), ("gate_dtype", C.c_int32), ("residual_bf16", C.c_void_p),
                ("next_norm_weight", C.c_void_p), ("next_norm_eps", C.c_float), ("next_normed_bf16", C.c_void_p),
                ("next_act_q", C.c_void_p), ("next_act_sf", C.c_void_p), ("hidden_q", C.c_void_p), ("hidden_sf", C.c_void_p)]


# name -> (restype, argtypes); exactly the entry points of include/vmoe.h
_P = C.c_void_p
SIGNATURES = {
    "vmoe_abi_version": (C.c_int, []),
    "vmoe_status_string": (C.c_char_p, [C.c_int]),
    "vmoe_workspace_bytes": (C.c_size_t, [C.POINTER(VmoeShape)]),
    "vmoe_workspace_layout": (C.c_int, [C.POINTER(VmoeShape), C.POINTER(VmoeWsLayout)]),
    "vmoe_route": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P]),
    "vmoe_build_tables": (C.c_int, [C.POINTER(VmoeShape), _P, _P, _P, C.c_int32, _P, C.c_size_t, _P]),
    "vmoe_quantize": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, _P]),
    "vmoe_prepare_sf": (C.c_int, [_P, C.c_int64, C.c_int32, _P, _P, _P]),
    "vmoe_dequantize": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int32, C.c_int64, _P, _P]),
    "vmoe_forward": (C.c_int, [C.POINTER(VmoeShape), C.POINTER(VmoeWeights), C.POINTER(VmoeWeights),
                               _P, _P, _P, _P, _P, _P, C.c_int32, _P, C.c_size_t, _P]),
    "vmoe_forward_ex": (C.c_int, [C.POINTER(VmoeShape), C.POINTER(VmoeWeights), C.POINTER(VmoeWeights),
                                  _P, _P, _P, _P, _P, _P, C.c_int32, _P, C.c_size_t, C.POINTER(VmoeExtras), _P]),
    "vmoe_rmsnorm_quantize": (C.c_int, [_P, _P, C.c_float, C.c_int32, C.c_int32, _P, _P, _P, _P]),
    "vmoe_router_gemv": (C.c_int, [_P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "vmoe_stage_gate_up": (C.c_int, [C.POINTER(VmoeShape), C.POINTER(VmoeWeights), C.POINTER(VmoeWeights),
                                     C.c_int32, _P, _P]),
    "vmoe_stage_down": (C.c_int, [C.POINTER(VmoeShape), C.POINTER(VmoeWeights), C.POINTER(VmoeWeights),
                                  C.c_int32, _P, _P]),
    "vmoe_stage_experts": (C.c_int, [C.POINTER(VmoeShape), C.POINTER(VmoeWeights), C.POINTER(VmoeWeights),
                                     C.c_int32, _P, _P]),
    "vmoe_stage_combine": (C.c_int, [C.POINTER(VmoeShape), C.c_int32, _P, _P, _P]),
    "vmoe_read_status": (C.c_int, [_P, C.POINTER(VmoeShape), _P]),
    "vmoe_ep_slab_bytes": (C.c_size_t, [C.POINTER(VmoeEpCtx), C.POINTER(VmoeShape)]),
    "vmoe_ep_workspace_bytes": (C.c_size_t, [C.POINTER(VmoeEpCtx), C.POINTER(VmoeShape)]),
    "vmoe_ep_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "vmoe_ep_free": (C.c_int, [_P]),
    "vmoe_ep_ipc_export": (C.c_int, [_P, _P]),
    "vmoe_ep_ipc_open": (C.c_int, [_P, C.POINTER(C.c_void_p)]),
    "vmoe_ep_ipc_close": (C.c_int, [_P]),
    "vmoe_ep_forward": (C.c_int, [C.POINTER(VmoeEpCtx), C.POINTER(VmoeShape), C.POINTER(VmoeWeights),
                                  C.POINTER(VmoeWeights), _P, _P, _P, _P, C.c_int32, _P, C.c_size_t, _P]),
    "vmoe_ep_read_status": (C.c_int, [C.POINTER(VmoeEpCtx), C.POINTER(VmoeShape), _P, _P]),
    "vmoe_permute_noalloc": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       _P, _P, _P, _P, _P, _P]),
}


class VmoeError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib.vmoe_status_string(status).decode() if "lib" in globals() else str(status)
        super().__init__(f"{where}: vmoe status {status} ({msg})")


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python sm120_moe_bench_b200/build.py` "
            "(there is no CPU or PyTorch fallback for this operator)")
    handle = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)          # AttributeError if a symbol is absent
        fn.restype = res
        fn.argtypes = args
    return handle


lib = _load()


def check(status: int, where: str) -> None:
    if status != 0:
        raise VmoeError(status, where)
