"""Expert parallelism across the GPUs of one box: host side.

One process per GPU.  ``torch.distributed`` is used once, at construction, to exchange the 64-byte
IPC handles of the per-rank slabs (the data path never calls a collective): afterwards every
forward is a chain of kernels on the caller's stream that write quantised token rows into the
owning rank's slab and weighted output rows back into the token owner's slab over NVLink.

Partition (fused-moe/p2p_moe_routing.py:26-33 of the reference): experts in contiguous blocks,
``gpu = e // (E // G)``, ``local = e % (E // G)``; the shared expert is replicated and computed by
the token's owner.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import ops
from ._lib import VmoeEpCtx, check, lib


def expert_partition(num_experts: int, world: int, rank: int):
    """``(first expert, experts per rank)`` of ``rank``; the expert count must divide evenly."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    per = num_experts // world
    return rank * per, per


def expert_map_for_rank(num_experts: int, world: int, rank: int) -> torch.Tensor:
    """The ``expert_map`` vector the reference's operator receives under expert parallelism
    (fused-moe/verdict_moe.py:473-477): local id for owned experts, -1 elsewhere."""
    first, per = expert_partition(num_experts, world, rank)
    m = torch.full((num_experts,), -1, dtype=torch.int32)
    m[first:first + per] = torch.arange(per, dtype=torch.int32)
    return m


def default_capacity(max_local_tokens: int, topk: int, world: int) -> int:
    """Rows one rank may send to one destination per call.  Worst case is every pair of every local
    token landing on the same rank (plus the shared-expert rows on the owner itself)."""
    return max_local_tokens * (topk + 1)


class ExpertParallelMoE:
    """The fused NVFP4 MoE layer with its experts split over the ranks of ``group``.

    ``routed`` holds this rank's ``E // G`` experts (prepared for the tensor-core path), ``shared``
    the replicated shared expert or ``None``.  ``forward(hidden, router_logits)`` takes this
    rank's own tokens (router logits over all ``E`` experts) and returns their combined output.
    """

    def __init__(self, hidden: int, inter: int, num_global_experts: int, topk: int,
                 routed: ops.MoEWeights, shared: ops.MoEWeights | None, max_local_tokens: int,
                 group=None, capacity: int | None = None, device=None, wait_limit_us: int = 0,
                 fake_world: int | None = None):
        """``wait_limit_us``: limit of every cross-GPU wait (0 = one second).  ``fake_world`` (tests of the
        time-out path only): this process plays rank 0 of that many ranks, the other ranks' slabs are local
        buffers that nobody ever signals."""
        import torch.distributed as dist
        self.group = group
        if fake_world:
            self.rank, self.world = 0, int(fake_world)
        elif dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        _, per = expert_partition(num_global_experts, self.world, self.rank)
        if routed.num_experts != per:
            raise ValueError(f"rank holds {routed.num_experts} experts, expected {per}")
        self.routed = routed.prepare()
        self.shared = shared.prepare() if shared is not None else None
        self.shape = ops.MoEShape(hidden, inter, per, topk, max_local_tokens, has_shared=shared is not None,
                                  num_global_experts=num_global_experts, path=2)
        self._cshape = self.shape.cstruct()
        self.capacity = capacity or default_capacity(max_local_tokens, topk, self.world)
        self.ctx = VmoeEpCtx()
        self.ctx.rank, self.ctx.world = self.rank, self.world
        self.ctx.experts_per_rank, self.ctx.capacity, self.ctx.max_local_tokens = per, self.capacity, max_local_tokens
        self.ctx.wait_limit_us = wait_limit_us          # 0 = one second
        for i in range(self.world):
            self.ctx.slab[i] = 1          # placeholder so that the size queries validate
        slab_bytes = lib.vmoe_ep_slab_bytes(C.byref(self.ctx), C.byref(self._cshape))
        ws_bytes = lib.vmoe_ep_workspace_bytes(C.byref(self.ctx), C.byref(self._cshape))
        if slab_bytes == 0 or ws_bytes == 0:
            raise ValueError("unsupported expert-parallel shape")
        self.slab_bytes, self.ws_bytes = slab_bytes, ws_bytes
        with torch.cuda.device(self.device):
            own = C.c_void_p()
            check(lib.vmoe_ep_alloc(slab_bytes, C.byref(own)), "vmoe_ep_alloc")
            self._own = own.value
            self._opened = []
            handle = (C.c_ubyte * 64)()
            check(lib.vmoe_ep_ipc_export(self._own, handle), "vmoe_ep_ipc_export")
            handles = [bytes(handle)]
            self._fake = []
            if fake_world:
                for i in range(1, self.world):
                    other = C.c_void_p()
                    check(lib.vmoe_ep_alloc(slab_bytes, C.byref(other)), "vmoe_ep_alloc")
                    self._fake.append(other.value)
                    self.ctx.slab[i] = other.value
                self.ctx.slab[0] = self._own
            elif self.world > 1:
                gathered = [None] * self.world
                dist.all_gather_object(gathered, bytes(handle), group=group)
                handles = gathered
            for i in range(self.world if not fake_world else 0):
                if i == self.rank:
                    self.ctx.slab[i] = self._own
                else:
                    buf = (C.c_ubyte * 64).from_buffer_copy(handles[i])
                    mapped = C.c_void_p()
                    check(lib.vmoe_ep_ipc_open(buf, C.byref(mapped)), "vmoe_ep_ipc_open")
                    self._opened.append(mapped.value)
                    self.ctx.slab[i] = mapped.value
            self.ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=self.device)
        if self.world > 1 and not fake_world:
            dist.barrier(group=group)     # every slab is mapped everywhere before the first forward

    def forward(self, hidden: torch.Tensor, router_logits: torch.Tensor, out: torch.Tensor | None = None,
                residual: torch.Tensor | None = None):
        """One expert-parallel pass over this rank's tokens; every rank must call it the same number of times.
        The call keeps its sequence number on the device, so it can be captured in a CUDA graph.  With
        ``residual`` the result is ``residual + layer(hidden)`` (may be the same tensor as ``out``)."""
        M = hidden.shape[0]
        if out is None:
            out = torch.empty_like(hidden)
        check(lib.vmoe_ep_forward(C.byref(self.ctx), C.byref(self._cshape), C.byref(self.routed.cstruct()),
                                  C.byref(self.shared.cstruct()) if self.shared is not None else None,
                                  hidden.data_ptr(), router_logits.data_ptr(),
                                  residual.data_ptr() if residual is not None else None, out.data_ptr(), M,
                                  self.ws.data_ptr(), self.ws_bytes, torch.cuda.current_stream().cuda_stream),
              "vmoe_ep_forward")
        return out

    def status(self) -> int:
        return lib.vmoe_ep_read_status(C.byref(self.ctx), C.byref(self._cshape), self.ws.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)

    def close(self):
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            lib.vmoe_ep_ipc_close(p)
        self._opened = []
        for p in self._fake:
            lib.vmoe_ep_free(p)
        self._fake = []
        if self._own:
            lib.vmoe_ep_free(self._own)
            self._own = None
