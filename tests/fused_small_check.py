"""Child process of tests/test_gpu_layer.py: prints one SHA-256 per case of the layer output (and of the routing
and permutation tables the call left in the workspace) for small batches.  The parent runs it once with the
fused small-batch launch and once with the separate kernels (VMOE_FUSED_SMALL=0) and compares the lines."""
import hashlib
import os
import sys

import torch

os.environ.setdefault("VMOE_NO_VLLM", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import sm120_moe_bench_b200 as vm  # noqa: E402
from sm120_moe_bench_b200 import ops, synth  # noqa: E402


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().cpu().numpy().tobytes())
    return h.hexdigest()


cases = [(synth.LayerConfig("mid", 512, 256, 12, 3, True), [1, 2, 5, 16]),
         (synth.CONFIG_TINY, [4]),
         (synth.LayerConfig("odd", 1024, 768, 40, 6, False), [3, 9])]        # inter / 256 odd: one k-block per down stage
for cfg, sizes in cases:
    layer = synth.make_layer(cfg, seed=2)
    routed = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare() if cfg.shared else None
    for M in sizes:
        ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=cfg.shared, path=2))
        h, l = (t.cuda() for t in synth.make_inputs(cfg, M, seed=40 + M))
        out = vm.fused_moe(h, routed, ws, router_logits=l, shared=shared)
        ids = ws.view("topk_ids", torch.int32, M * cfg.topk).clone()
        w = ws.view("topk_weights", torch.float32, M * cfg.topk).clone()
        slots = ws.view("pair_slot", torch.int32, M * cfg.topk).clone()
        # pre-routed entry, residual, repeated call on the same workspace
        out2 = vm.fused_moe(h, routed, ws, topk_ids=ids.view(M, cfg.topk), topk_weights=w.view(M, cfg.topk), shared=shared,
                            residual=h)
        out3 = vm.fused_moe(h, routed, ws, router_logits=l, shared=shared)
        torch.cuda.synchronize()
        assert ws.status() == 0
        assert torch.equal(out, out3)
        print(cfg.name, M, digest(out, ids, w, slots, out2))
