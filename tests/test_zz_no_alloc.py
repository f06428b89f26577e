"""The allocation-free permutation entry point (vmoe_permute_noalloc) against the workspace-based
one (vmoe_build_tables), through the C ABI.

Some users of the library cannot allocate device memory when they call it -- a serving worker
whose pool already takes the whole GPU, a small FFI binding that owns no allocator -- so this
entry point keeps its scratch in a fixed array inside the library.  The test calls it twice in a
row with different inputs (the shared array keeps the previous call's contents, so the second
call proves it is cleared properly) and asks for identical tables.  The file name makes pytest
collect it after every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tables_both_ways(M, E, T, shared, seed, split=None):
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200._lib import lib
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(M, E, generator=g).cuda()
    ids, w = vm.route(logits, T)
    emap = None
    e_local = E
    if split is not None:
        lo, hi = split
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[lo:hi] = torch.arange(hi - lo, dtype=torch.int32)
        emap = emap.cuda()
        e_local = hi - lo
    # existing entry point: tables inside a workspace the caller allocated
    ws = vm.Workspace(vm.MoEShape(1024, 512, e_local, T, M, has_shared=shared, num_global_experts=E))
    vm.build_tables(ws, ids, w, emap)
    torch.cuda.synchronize()
    ref = ws.tables(M)
    # new entry point: only inputs and outputs are passed
    S = M * T + (M if shared else 0)
    out = dict(expert_offsets=torch.full((e_local + 2,), -7, dtype=torch.int32, device="cuda"),
               sorted_pair=torch.full((S,), -7, dtype=torch.int32, device="cuda"),
               pair_slot=torch.full((M * T,), -7, dtype=torch.int32, device="cuda"),
               gather_idx=torch.full((S,), -7, dtype=torch.int32, device="cuda"),
               scatter_weights=torch.full((S,), -7.0, dtype=torch.float32, device="cuda"))
    rc = lib.vmoe_permute_noalloc(ids.data_ptr(), w.data_ptr(), emap.data_ptr() if emap is not None else None,
                                  M, T, e_local, int(shared), out["expert_offsets"].data_ptr(),
                                  out["sorted_pair"].data_ptr(), out["pair_slot"].data_ptr(),
                                  out["gather_idx"].data_ptr(), out["scatter_weights"].data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    n = ref["num_slots"]
    assert torch.equal(out["expert_offsets"].cpu(), ref["expert_offsets"])
    assert torch.equal(out["pair_slot"].cpu(), ref["pair_slot"])
    for k in ("sorted_pair", "gather_idx", "scatter_weights"):
        assert torch.equal(out[k].cpu()[:n], ref[k]), k      # integer / copied-float tables: bit-exact


def test_no_alloc_matches_workspace_version_twice_in_a_row():
    _tables_both_ways(64, 512, 10, True, seed=1)
    _tables_both_ways(37, 512, 10, True, seed=2)            # smaller problem right after a larger one
    _tables_both_ways(1024, 256, 8, False, seed=3, split=(64, 192))
    _tables_both_ways(5, 16, 2, False, seed=4)


def test_no_alloc_rejects_sizes_beyond_the_fixed_maximum():
    from sm120_moe_bench_b200._lib import lib
    d = torch.zeros(16, dtype=torch.int32, device="cuda")
    f = torch.zeros(16, dtype=torch.float32, device="cuda")
    args = lambda M, E: (d.data_ptr(), f.data_ptr(), None, M, 2, E, 0, d.data_ptr(), d.data_ptr(), d.data_ptr(),
                         d.data_ptr(), f.data_ptr(), None)
    assert lib.vmoe_permute_noalloc(*args(1025, 8)) == 8      # VMOE_ERR_LIMIT
    assert lib.vmoe_permute_noalloc(*args(4, 1025)) == 8
    assert lib.vmoe_status_string(8).startswith(b"size beyond a fixed maximum")
