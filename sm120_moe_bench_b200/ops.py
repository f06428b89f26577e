"""Torch-facing wrappers of the C ABI.  Torch supplies device memory and the current stream;
all arithmetic happens in ``libvmoe.so``.  Nothing here allocates inside a forward call except
when the caller does not pass an output tensor.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import VmoeExtras, VmoeShape, VmoeWeights, VmoeWsLayout, check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


@dataclass(frozen=True)
class MoEShape:
    hidden: int
    inter: int
    num_experts: int          # experts held by this GPU
    topk: int
    max_tokens: int
    has_shared: bool = False
    num_global_experts: int | None = None
    path: int = 0             # 0 automatic, 1 streaming GEMV (CUDA cores), 2 tcgen05 tensor cores

    def cstruct(self) -> VmoeShape:
        return VmoeShape(self.hidden, self.inter, self.num_experts, self.topk, self.max_tokens,
                         int(self.has_shared), self.num_global_experts or self.num_experts, self.path)


class MoEWeights:
    """NVFP4 expert weights in the reference's layout (fused-moe/verdict_moe.py:571-575):
    ``w13 [E, 2N, K/2]`` u8, ``w13_sf [E, 2N, K/16]`` u8 (or float8_e4m3fn, viewed as bytes as
    fused-moe/verdict_moe.py:519-520 does), ``w13_gs [E]`` f32, ``w2 [E, K, N/2]``,
    ``w2_sf [E, K, N/16]``, ``w2_gs [E]``."""

    def __init__(self, w13, w13_sf, w13_gs, w2, w2_sf, w2_gs):
        as_u8 = lambda t: t.view(torch.uint8) if t.dtype != torch.uint8 else t
        self.w13 = _need(as_u8(w13), torch.uint8, "w13")
        self.w13_sf = _need(as_u8(w13_sf), torch.uint8, "w13_sf")
        self.w13_gs = _need(w13_gs, torch.float32, "w13_gs")
        self.w2 = _need(as_u8(w2), torch.uint8, "w2")
        self.w2_sf = _need(as_u8(w2_sf), torch.uint8, "w2_sf")
        self.w2_gs = _need(w2_gs, torch.float32, "w2_gs")
        E, N2, Kh = self.w13.shape
        if self.w13_sf.shape != (E, N2, Kh // 8) or self.w2.shape != (E, Kh * 2, N2 // 4) \
                or self.w2_sf.shape != (E, Kh * 2, N2 // 32) or self.w13_gs.numel() != E or self.w2_gs.numel() != E:
            raise ValueError("inconsistent NVFP4 weight shapes")
        self.w13_sf_atoms = None
        self.w2_sf_atoms = None
        self._c = VmoeWeights(self.w13.data_ptr(), self.w13_sf.data_ptr(), self.w13_gs.data_ptr(),
                              self.w2.data_ptr(), self.w2_sf.data_ptr(), self.w2_gs.data_ptr(), None, None)

    def prepare(self) -> "MoEWeights":
        """One-time re-layout of the block scales for the tensor-core path (``vmoe_prepare_sf``);
        raises if a scale byte has its sign bit set.  Needs 2N and K to be multiples of 128."""
        if self.w13_sf_atoms is not None:
            return self
        bad = torch.zeros(1, dtype=torch.int32, device=self.w13.device)
        outs = []
        for sf in (self.w13_sf, self.w2_sf):
            E, R, C16 = sf.shape
            atoms = torch.empty(sf.numel(), dtype=torch.uint8, device=sf.device)
            check(lib.vmoe_prepare_sf(sf.data_ptr(), E * R, C16 * 16, atoms.data_ptr(), bad.data_ptr(), _stream()),
                  "vmoe_prepare_sf")
            outs.append(atoms)
        if int(bad.item()) != 0:
            raise ValueError(f"{int(bad.item())} block-scale bytes have the sign bit set; NVFP4 scales are unsigned")
        self.w13_sf_atoms, self.w2_sf_atoms = outs
        self._c.w13_sf_atoms = self.w13_sf_atoms.data_ptr()
        self._c.w2_sf_atoms = self.w2_sf_atoms.data_ptr()
        return self

    num_experts = property(lambda self: self.w13.shape[0])
    hidden = property(lambda self: self.w13.shape[2] * 2)
    inter = property(lambda self: self.w13.shape[1] // 2)

    def cstruct(self) -> VmoeWeights:
        return self._c

    def nbytes_per_expert(self) -> int:
        return (self.w13[0].numel() + self.w13_sf[0].numel() + self.w2[0].numel() + self.w2_sf[0].numel())


class Workspace:
    """Caller-owned scratch blob of ``vmoe_workspace_bytes`` bytes, zero-initialised once.
    Plays the part of the reference's ``setup_buffers`` pool (fused-moe/verdict_moe.py:243-414)."""

    def __init__(self, shape: MoEShape, device="cuda"):
        self.shape = shape
        self._cshape = shape.cstruct()
        layout = VmoeWsLayout()
        check(lib.vmoe_workspace_layout(C.byref(self._cshape), C.byref(layout)), "vmoe_workspace_layout")
        self.layout = {n: getattr(layout, n) for n, _ in VmoeWsLayout._fields_}
        self.nbytes = self.layout["total_bytes"]
        assert self.nbytes == lib.vmoe_workspace_bytes(C.byref(self._cshape))
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)

    def view(self, name: str, dtype: torch.dtype, numel: int) -> torch.Tensor:
        off = self.layout[name]
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self.buf[off:off + nbytes].view(dtype)

    def status(self) -> int:
        return lib.vmoe_read_status(self.buf.data_ptr(), C.byref(self._cshape), _stream())

    # decoded views of the tables for M tokens (tests, debugging)
    def tables(self, M: int) -> dict:
        s = self.shape
        P = M * s.topk
        cnt = self.view("counters", torch.int32, 8).cpu()
        slots = int(cnt[1])
        return dict(
            expert_offsets=self.view("expert_offsets", torch.int32, s.num_experts + 2).cpu(),
            sorted_pair=self.view("sorted_pair", torch.int32, slots).cpu(),
            pair_slot=self.view("pair_slot", torch.int32, P).cpu(),
            gather_idx=self.view("gather_idx", torch.int32, slots).cpu(),
            scatter_weights=self.view("scatter_weights", torch.float32, slots).cpu(),
            num_units=int(cnt[0]), num_slots=slots,
            units=self.view("units", torch.int32, int(cnt[0]) * 4).cpu().view(-1, 4),
            num_tc_units=int(cnt[5]),
            tc_units=self.view("tc_units", torch.int32, int(cnt[5]) * 4).cpu().view(-1, 4),
        )


def route(logits: torch.Tensor, topk: int):
    """Softmax / top-k / renormalise on the device.  Returns ``(ids int32 [M, T], weights f32 [M, T])``."""
    _need(logits, torch.float32, "logits")
    M, E = logits.shape
    ids = torch.empty(M, topk, dtype=torch.int32, device=logits.device)
    w = torch.empty(M, topk, dtype=torch.float32, device=logits.device)
    check(lib.vmoe_route(logits.data_ptr(), M, E, topk, ids.data_ptr(), w.data_ptr(), _stream()), "vmoe_route")
    return ids, w


def build_tables(ws: Workspace, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                 expert_map: torch.Tensor | None = None) -> None:
    _need(topk_ids, torch.int32, "topk_ids")
    _need(topk_weights, torch.float32, "topk_weights")
    if expert_map is not None:
        _need(expert_map, torch.int32, "expert_map")
    M = topk_ids.shape[0]
    check(lib.vmoe_build_tables(C.byref(ws._cshape), topk_ids.data_ptr(), topk_weights.data_ptr(),
                                _ptr(expert_map), M, ws.buf.data_ptr(), ws.nbytes, _stream()),
          "vmoe_build_tables")


def quantize(x: torch.Tensor):
    """bf16 ``[rows, K]`` -> (packed u8 ``[rows, K/2]``, block scales u8 ``[rows, K/16]``)."""
    _need(x, torch.bfloat16, "x")
    rows, K = x.shape
    packed = torch.empty(rows, K // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(rows, K // 16, dtype=torch.uint8, device=x.device)
    check(lib.vmoe_quantize(x.data_ptr(), rows, K, packed.data_ptr(), sf.data_ptr(), _stream()), "vmoe_quantize")
    return packed, sf


def dequantize(packed: torch.Tensor, sf: torch.Tensor, global_scale: torch.Tensor | None = None,
               rows_per_scale: int = 1) -> torch.Tensor:
    """NVFP4 -> f32; ``global_scale[i]`` applies to rows ``[i*rows_per_scale, (i+1)*rows_per_scale)``."""
    _need(packed, torch.uint8, "packed")
    _need(sf, torch.uint8, "sf")
    K = packed.shape[-1] * 2
    rows = packed.numel() // (K // 2)
    out = torch.empty(*packed.shape[:-1], K, dtype=torch.float32, device=packed.device)
    check(lib.vmoe_dequantize(packed.data_ptr(), sf.data_ptr(), _ptr(global_scale), rows, K,
                              rows_per_scale, out.data_ptr(), _stream()), "vmoe_dequantize")
    return out


def fused_moe(hidden: torch.Tensor, weights: MoEWeights, ws: Workspace, *,
              router_logits: torch.Tensor | None = None,
              topk_ids: torch.Tensor | None = None, topk_weights: torch.Tensor | None = None,
              shared: MoEWeights | None = None, expert_map: torch.Tensor | None = None,
              out: torch.Tensor | None = None, gate_weight: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, hidden_quantized: "QuantizedRows | None" = None,
              next_norm: "tuple[torch.Tensor, float] | None" = None,
              next_rows: "QuantizedRows | None" = None) -> torch.Tensor:
    """The fused NVFP4 MoE expert layer: bf16 hidden states + router logits (or pre-routed
    ids / weights, or the router matrix ``gate_weight [E, K]`` f32 / bf16 for the projection to run
    on the device too) + packed expert weights in, combined bf16 out.  With ``residual`` the result
    is ``residual + layer(hidden)`` (may be the same tensor as ``out``).

    ``next_norm = (gamma f32 [K], eps)`` fuses the next layer's RMSNorm and activation quantisation behind the
    combine: ``next_rows`` (a ``QuantizedRows``) receives the normalised bf16 rows, their FP4 codes and block
    scales.  ``hidden_quantized`` feeds such rows to this layer in place of quantising ``hidden`` again."""
    if hidden is None:
        if hidden_quantized is None:
            raise ValueError("hidden or hidden_quantized is required")
        M, K = hidden_quantized.packed.shape[0], hidden_quantized.packed.shape[1] * 2
    else:
        _need(hidden, torch.bfloat16, "hidden")
        M, K = hidden.shape
    if out is None:
        out = torch.empty(M, K, dtype=torch.bfloat16, device=(hidden if hidden is not None else hidden_quantized.packed).device)
    else:
        _need(out, torch.bfloat16, "out")
    extras = None
    if router_logits is not None:
        _need(router_logits, torch.float32, "router_logits")
    elif gate_weight is not None and topk_ids is None:
        if gate_weight.dtype not in (torch.float32, torch.bfloat16) or not gate_weight.is_contiguous():
            raise TypeError("gate_weight must be a contiguous f32 or bf16 tensor [E, K]")
        extras = VmoeExtras()
        extras.gate_weight = gate_weight.data_ptr()
        extras.gate_dtype = 0 if gate_weight.dtype == torch.float32 else 1
    else:
        _need(topk_ids, torch.int32, "topk_ids")
        _need(topk_weights, torch.float32, "topk_weights")
    if residual is not None:
        _need(residual, torch.bfloat16, "residual")
        if extras is None:
            extras = VmoeExtras()
        extras.residual_bf16 = residual.data_ptr()
    if hidden_quantized is not None:
        if extras is None:
            extras = VmoeExtras()
        extras.hidden_q = _need(hidden_quantized.packed, torch.uint8, "hidden_quantized.packed").data_ptr()
        extras.hidden_sf = _need(hidden_quantized.sf, torch.uint8, "hidden_quantized.sf").data_ptr()
    if next_norm is not None:
        if next_rows is None:
            raise ValueError("next_norm needs next_rows to write to")
        gamma, eps = next_norm
        if extras is None:
            extras = VmoeExtras()
        extras.next_norm_weight = _need(gamma, torch.float32, "gamma").data_ptr()
        extras.next_norm_eps = float(eps)
        extras.next_normed_bf16 = _ptr(next_rows.normed)
        extras.next_act_q = next_rows.packed.data_ptr()
        extras.next_act_sf = next_rows.sf.data_ptr()
    if expert_map is not None:
        _need(expert_map, torch.int32, "expert_map")
    if ws.shape.has_shared and shared is None:
        raise ValueError("shape has a shared expert but no shared weights were given")
    check(lib.vmoe_forward_ex(C.byref(ws._cshape), C.byref(weights.cstruct()),
                              C.byref(shared.cstruct()) if shared is not None else None,
                              _ptr(hidden), _ptr(router_logits), _ptr(topk_ids), _ptr(topk_weights),
                              _ptr(expert_map), out.data_ptr(), M, ws.buf.data_ptr(), ws.nbytes,
                              C.byref(extras) if extras is not None else None, _stream()),
          "vmoe_forward_ex")
    return out


class QuantizedRows:
    """Normalised activation rows as a layer's fused epilogue (or ``rmsnorm_quantize``) leaves them for the next
    layer: bf16 rows ``[M, K]`` (optional), E2M1 codes ``[M, K/2]`` and E4M3 block scales ``[M, K/16]``."""

    def __init__(self, rows: int, K: int, device="cuda", keep_bf16: bool = True):
        self.normed = torch.empty(rows, K, dtype=torch.bfloat16, device=device) if keep_bf16 else None
        self.packed = torch.empty(rows, K // 2, dtype=torch.uint8, device=device)
        self.sf = torch.empty(rows, K // 16, dtype=torch.uint8, device=device)


def rmsnorm_quantize(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, out: QuantizedRows | None = None) -> QuantizedRows:
    """``y = bf16(x * rsqrt(mean(x^2) + eps) * gamma)`` per row, then ``y`` quantised to NVFP4 (``vmoe_rmsnorm_quantize``)."""
    _need(x, torch.bfloat16, "x")
    _need(gamma, torch.float32, "gamma")
    rows, K = x.shape
    out = out or QuantizedRows(rows, K, x.device)
    check(lib.vmoe_rmsnorm_quantize(x.data_ptr(), gamma.data_ptr(), float(eps), rows, K, _ptr(out.normed),
                                    out.packed.data_ptr(), out.sf.data_ptr(), _stream()), "vmoe_rmsnorm_quantize")
    return out


def router_gemv(hidden: torch.Tensor, gate_weight: torch.Tensor) -> torch.Tensor:
    """``hidden [M, K] bf16 @ gate_weight [E, K]^T`` -> f32 logits ``[M, E]`` (fixed summation order)."""
    _need(hidden, torch.bfloat16, "hidden")
    if gate_weight.dtype not in (torch.float32, torch.bfloat16) or not gate_weight.is_contiguous():
        raise TypeError("gate_weight must be a contiguous f32 or bf16 tensor [E, K]")
    M, K = hidden.shape
    E = gate_weight.shape[0]
    logits = torch.empty(M, E, dtype=torch.float32, device=hidden.device)
    check(lib.vmoe_router_gemv(hidden.data_ptr(), gate_weight.data_ptr(), 0 if gate_weight.dtype == torch.float32 else 1,
                               M, K, E, logits.data_ptr(), _stream()), "vmoe_router_gemv")
    return logits


def run_stage(name: str, ws: Workspace, weights: MoEWeights, shared: MoEWeights | None, M: int,
              out: torch.Tensor | None = None) -> None:
    """Run one stage (``gate_up`` / ``down`` / ``experts`` = both in the forward's own launch(es) / ``combine``) over
    an already built workspace."""
    sh = C.byref(shared.cstruct()) if shared is not None else None
    if name == "gate_up":
        check(lib.vmoe_stage_gate_up(C.byref(ws._cshape), C.byref(weights.cstruct()), sh, M,
                                     ws.buf.data_ptr(), _stream()), "vmoe_stage_gate_up")
    elif name == "down":
        check(lib.vmoe_stage_down(C.byref(ws._cshape), C.byref(weights.cstruct()), sh, M,
                                  ws.buf.data_ptr(), _stream()), "vmoe_stage_down")
    elif name == "experts":
        check(lib.vmoe_stage_experts(C.byref(ws._cshape), C.byref(weights.cstruct()), sh, M,
                                     ws.buf.data_ptr(), _stream()), "vmoe_stage_experts")
    elif name == "combine":
        check(lib.vmoe_stage_combine(C.byref(ws._cshape), M, ws.buf.data_ptr(), out.data_ptr(), _stream()),
              "vmoe_stage_combine")
    else:
        raise ValueError(name)
