"""Test infrastructure, not part of the product: ctypes view of ``oracle/_ref/libref_host.so``, the reference's
own host C++ reference compiled by ``oracle/build_ref.py`` (fused-moe/csrc/verdict_fused_independent.cu:50-86,
474-564).  ``load()`` returns None when the library has not been built."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

LIB = Path(__file__).resolve().parent / "_ref" / "libref_host.so"
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


class RefHost:
    def __init__(self, lib: C.CDLL):
        self.lib = lib
        lib.ref_hidden.restype = C.c_int
        lib.ref_e4m3_decode.restype = C.c_float; lib.ref_e4m3_decode.argtypes = [C.c_ubyte]
        lib.ref_e4m3_encode.restype = C.c_ubyte; lib.ref_e4m3_encode.argtypes = [C.c_float]
        lib.ref_e4m3_encode_ceil.restype = C.c_ubyte; lib.ref_e4m3_encode_ceil.argtypes = [C.c_float]
        lib.ref_silu.restype = C.c_float; lib.ref_silu.argtypes = [C.c_float]
        lib.ref_quantize.restype = None; lib.ref_quantize.argtypes = [_f32p, C.c_int, _u8p, _u8p]
        lib.ref_dequant.restype = C.c_float; lib.ref_dequant.argtypes = [_u8p, _u8p, C.c_int]
        lib.ref_layer_single.restype = None
        lib.ref_layer_single.argtypes = [_u8p, _u8p, _u8p, _u8p, _u8p, _u8p, _i32p, _f32p, _f32p, C.c_int, C.c_int]
        self.hidden = int(lib.ref_hidden())

    def e4m3_decode_all(self) -> np.ndarray:
        return np.array([self.lib.ref_e4m3_decode(b) for b in range(256)], dtype=np.float32)

    def e4m3_encode(self, x) -> np.ndarray:
        return np.array([self.lib.ref_e4m3_encode(float(v)) for v in np.asarray(x, np.float32).ravel()], dtype=np.uint8)

    def e4m3_encode_ceil(self, x) -> np.ndarray:
        return np.array([self.lib.ref_e4m3_encode_ceil(float(v)) for v in np.asarray(x, np.float32).ravel()], dtype=np.uint8)

    def quantize(self, data: np.ndarray):
        """quantize_to_nvfp4_e4m3: flat float32, 16-element blocks -> (packed u8 [n/2], scales u8 [n/16])."""
        d = np.ascontiguousarray(data, dtype=np.float32).ravel()
        packed = np.zeros(d.size // 2, np.uint8); sf = np.zeros(d.size // 16, np.uint8)
        self.lib.ref_quantize(d, d.size, packed, sf)
        return packed, sf

    def dequantize(self, packed: np.ndarray, sf: np.ndarray) -> np.ndarray:
        p = np.ascontiguousarray(packed, np.uint8).ravel(); s = np.ascontiguousarray(sf, np.uint8).ravel()
        return np.array([self.lib.ref_dequant(p, s, i) for i in range(p.size * 2)], dtype=np.float32)

    def layer_single(self, x_packed, x_sf, w13, w13_sf, w2, w2_sf, expert_ids, expert_weights) -> np.ndarray:
        """host_quantized_reference_single: one quantised token row of ``hidden`` elements through the listed
        experts (``w13 [E, 2N, K/2]``, ``w2 [E, K, N/2]`` and their linear block scales; no global scales)."""
        n_half = w13.shape[1] // 2
        out = np.zeros(self.hidden, np.float32)
        ids = np.ascontiguousarray(expert_ids, np.int32); wts = np.ascontiguousarray(expert_weights, np.float32)
        self.lib.ref_layer_single(np.ascontiguousarray(x_packed, np.uint8).ravel(), np.ascontiguousarray(x_sf, np.uint8).ravel(),
                                  np.ascontiguousarray(w13, np.uint8).ravel(), np.ascontiguousarray(w13_sf, np.uint8).ravel(),
                                  np.ascontiguousarray(w2, np.uint8).ravel(), np.ascontiguousarray(w2_sf, np.uint8).ravel(),
                                  ids, wts, out, int(ids.size), int(n_half))
        return out


def load() -> RefHost | None:
    if not LIB.exists():
        return None
    return RefHost(C.CDLL(str(LIB)))


# ---------------------------------------------------------------------------------------------
# The reference's host permutation (build_group_tables, fused-moe/csrc/verdict_fused_grouped.cu:655-691)
# and its router (moe_topk_select, fused-moe/csrc/megakernel_v1.cu:491-537), compiled by build_ref.py.
# ---------------------------------------------------------------------------------------------
LIB_TABLES = LIB.parent / "libref_tables.so"
LIB_ROUTER = LIB.parent / "libref_router.so"


class RefTables:
    ROW = 10          # the reference's routing rows are ten experts wide

    def __init__(self, lib: C.CDLL):
        self.lib = lib
        lib.ref_build_group_tables.restype = C.c_int
        lib.ref_build_group_tables.argtypes = [_i32p, C.c_int, C.c_int, C.c_float, _i32p, _i32p, _i32p, _i32p, _f32p]

    def build_group_tables(self, topk_ids: np.ndarray, weight: float = 1.0) -> dict:
        """``topk_ids [M, T]`` (T <= 10) -> the reference's GroupTables as arrays.  The reference gives every
        pair the same weight."""
        ids = np.asarray(topk_ids, np.int32)
        M, T = ids.shape
        assert T <= self.ROW
        rows = np.zeros((M, self.ROW), np.int32)
        rows[:, :T] = ids
        P = M * T
        el, cnt, off = np.zeros(P, np.int32), np.zeros(P, np.int32), np.zeros(P + 1, np.int32)
        gi, sw = np.zeros(P, np.int32), np.zeros(P, np.float32)
        g = int(self.lib.ref_build_group_tables(rows, M, T, float(weight), el, cnt, off, gi, sw))
        return dict(expert_list=el[:g], expert_token_count=cnt[:g], expert_token_offset=off[:g + 1],
                    gather_idx=gi, scatter_weights=sw)


class RefRouter:
    def __init__(self, lib: C.CDLL):
        self.lib = lib
        lib.ref_topk_select.restype = None
        lib.ref_topk_select.argtypes = [_f32p, C.c_int, C.c_int, _i32p, _f32p, _f32p]

    def route(self, logits: np.ndarray, topk: int):
        """Row by row through the reference's moe_topk_select -> ``(ids int32 [M, T], weights f32 [M, T])``."""
        lg = np.ascontiguousarray(logits, np.float32)
        M, E = lg.shape
        ids, w = np.zeros((M, topk), np.int32), np.zeros((M, topk), np.float32)
        scratch = np.zeros(E, np.float32)
        for m in range(M):
            self.lib.ref_topk_select(lg[m], E, topk, ids[m], w[m], scratch)
        return ids, w


def load_tables() -> RefTables | None:
    return RefTables(C.CDLL(str(LIB_TABLES))) if LIB_TABLES.exists() else None


def load_router() -> RefRouter | None:
    return RefRouter(C.CDLL(str(LIB_ROUTER))) if LIB_ROUTER.exists() else None
