"""GPU parity, stage by stage, through the C ABI: router (a1), permutation tables (a3, a4),
activation quantiser (a6) and decoder (a7) must match the oracle bit for bit."""
import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import nvfp4

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vm():
    import sm120_moe_bench_b200 as pkg
    return pkg


def _logits(M, E, seed, zipf=None):
    g = torch.Generator().manual_seed(seed)
    l = torch.randn(M, E, generator=g)
    if zipf:
        perm = torch.randperm(E, generator=g)
        rank = torch.empty(E); rank[perm] = torch.arange(1, E + 1, dtype=torch.float32)
        l = l - zipf * torch.log(rank)
    return l.float().contiguous()


@pytest.mark.parametrize("M,E,T,zipf", [(4, 8, 2, None), (1, 512, 10, None), (64, 512, 10, None),
                                        (1536, 512, 10, 1.2), (8192, 512, 10, None), (33, 160, 6, None),
                                        (7, 40, 16, None), (9, 1000, 8, None), (5, 2048, 10, None)])
def test_route_matches_oracle(vm, M, E, T, zipf):
    l = _logits(M, E, 1234 + M, zipf)
    assert omoe.route_ids_are_unambiguous(l.numpy(), T)
    ids_ref, w_ref = omoe.route(l.numpy(), T)
    ids, w = vm.route(l.cuda(), T)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)                     # bit-exact ids and order
    np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=2e-6, atol=0)  # expf / sum-order last bits
    np.testing.assert_allclose(w.cpu().numpy().sum(1), 1.0, rtol=1e-6)


def test_route_ties_lowest_id_wins(vm):
    l = torch.zeros(3, 64)
    l[1, 10] = l[1, 50] = 2.0          # two equal maxima
    l[2, 5:9] = 1.0
    ids, w = vm.route(l.cuda(), 4)
    ids_ref, w_ref = omoe.route(l.numpy(), 4)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert ids.cpu().numpy()[0].tolist() == [0, 1, 2, 3]
    assert ids.cpu().numpy()[1].tolist()[:2] == [10, 50]
    assert ids.cpu().numpy()[2].tolist() == [5, 6, 7, 8]


def _check_tables(vm, M, E, T, shared, emap_split=None, seed=0):
    l = _logits(M, E, seed)
    ids_ref, w_ref = omoe.route(l.numpy(), T)
    ids = torch.from_numpy(ids_ref).cuda(); w = torch.from_numpy(w_ref).cuda()
    if emap_split is None:
        e_local, emap_t, keep, local_ids = E, None, None, ids_ref
    else:
        lo, hi = emap_split
        emap = np.full(E, -1, np.int32); emap[lo:hi] = np.arange(hi - lo, dtype=np.int32)
        e_local, emap_t = hi - lo, torch.from_numpy(emap).cuda()
        keep = emap[ids_ref] >= 0
        local_ids = np.maximum(emap[ids_ref], 0)
    shape = vm.MoEShape(1024, 512, e_local, T, max(M, 1), has_shared=shared, num_global_experts=E)
    ws = vm.Workspace(shape)
    vm.build_tables(ws, ids, w, emap_t)
    torch.cuda.synchronize()
    t = ws.tables(M)
    ref = omoe.build_group_tables(local_ids, w_ref, e_local, keep)
    P_kept = ref.sorted_pair.size
    off = t["expert_offsets"].numpy()
    assert np.array_equal(off[: e_local + 1], ref.expert_offsets)
    assert t["num_slots"] == P_kept + (M if shared else 0)
    assert np.array_equal(t["sorted_pair"].numpy()[:P_kept], ref.sorted_pair)
    assert np.array_equal(t["gather_idx"].numpy()[:P_kept], ref.gather_idx)
    assert np.array_equal(t["scatter_weights"].numpy()[:P_kept], ref.scatter_weights)
    assert np.array_equal(t["pair_slot"].numpy(), ref.pair_slot)
    if shared:
        assert np.array_equal(t["gather_idx"].numpy()[P_kept:], np.arange(M))
        assert np.all(t["scatter_weights"].numpy()[P_kept:] == 1.0)
        assert off[e_local + 1] == P_kept + M
    # work units cover every slot exactly once, <= 4 tokens each, never crossing an expert
    units = t["units"].numpy()
    covered = np.zeros(t["num_slots"], np.int32)
    bounds = np.concatenate([ref.expert_offsets, [t["num_slots"]]])
    for e, s0, n, _ in units:
        assert 1 <= n <= 4 and bounds[e] <= s0 and s0 + n <= bounds[e + 1]
        covered[s0:s0 + n] += 1
    assert np.all(covered == 1)


@pytest.mark.parametrize("M,E,T,shared", [(4, 8, 2, False), (1, 512, 10, True), (64, 512, 10, True),
                                          (1536, 512, 10, True), (8192, 512, 10, True), (100, 40, 16, False)])
def test_tables_match_oracle(vm, M, E, T, shared):
    _check_tables(vm, M, E, T, shared)


def test_tables_expert_map(vm):
    _check_tables(vm, 64, 512, 10, True, emap_split=(128, 256))
    _check_tables(vm, 3000, 512, 10, False, emap_split=(448, 512))


def test_quantize_bit_exact(vm):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(37, 1024, generator=g)
    x[0, :16] = 0.0                                   # zero block -> scale byte 0, codes 0
    x[1, :32] *= 1e4                                   # saturating scales (amax/6 > 448)
    x[2, :32] *= 1e-6                                  # sub-normal E4M3 scales
    x[3, :16] = torch.tensor([6, 5, 3.5, 2.5, 1.75, 1.25, .75, .25, -6, -5, -3.5, -2.5, -1.75, -1.25, -.75, -.25])
    x[4, :16] = -0.0
    xb = x.to(torch.bfloat16)
    packed, sf = vm.quantize(xb.cuda())
    p_ref, s_ref = nvfp4.quantize_act(xb.float().numpy())
    assert np.array_equal(sf.cpu().numpy(), s_ref)
    assert np.array_equal(packed.cpu().numpy(), p_ref)


def test_quantize_large(vm):
    g = torch.Generator().manual_seed(6)
    xb = (torch.randn(512, 4096, generator=g) * 3).to(torch.bfloat16)
    packed, sf = vm.quantize(xb.cuda())
    p_ref, s_ref = nvfp4.quantize_act(xb.float().numpy())
    assert np.array_equal(sf.cpu().numpy(), s_ref) and np.array_equal(packed.cpu().numpy(), p_ref)


def test_dequantize_all_codes_all_scales(vm):
    # every scale byte (incl. the NaN patterns, which decode to 0, and negative bytes) x every code
    sf = torch.arange(256, dtype=torch.uint8).view(256, 1)
    codes = torch.arange(16, dtype=torch.uint8)
    packed = (codes[0::2] | (codes[1::2] << 4)).view(1, 8).repeat(256, 1).contiguous()
    out = vm.dequantize(packed.cuda(), sf.cuda())
    ref = nvfp4.dequantize(packed.numpy(), sf.numpy())
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    gs = torch.tensor([0.5, 3.0], dtype=torch.float32)
    out = vm.dequantize(packed.cuda(), sf.cuda(), gs.cuda(), rows_per_scale=128)
    ref2 = ref * np.repeat(gs.numpy(), 128)[:, None]
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref2.astype(np.float32).view(np.uint32))


def test_argument_errors(vm):
    from sm120_moe_bench_b200._lib import VmoeError
    with pytest.raises(VmoeError):
        vm.route(torch.zeros(2, 4, device="cuda"), 5)          # T > E
    with pytest.raises(VmoeError):
        vm.Workspace(vm.MoEShape(1000, 512, 8, 2, 4))          # K not a multiple of 128
    with pytest.raises(ValueError):
        vm.quantize(torch.zeros(2, 64, device="cuda"))         # not bf16
