"""Development aid: where the time of a small decode step goes, from ``%globaltimer`` marks inside the kernels.

Needs the library built with the marks compiled in::

    VMOE_TIMELINE=1 python sm120_moe_bench_b200/build.py --force
    python -m sm120_moe_bench_b200.timeline [batch sizes ...]

(an ordinary build has no marks at all and this module refuses to run).  For every batch size it runs the config-2
layer a few times and prints, for two steps on fresh inputs, the marks in microseconds relative to the first one:
when the fused kernel's CTAs started, had TMEM, passed the dependency on the front kernel, knew the unit count, saw
their first complete ring stage, issued the last gate_up stage / the first down stage, and when the last CTA left.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

os.environ.setdefault("VMOE_NO_VLLM", "1")

NAMES = {8: "fused kernel entry (first CTA)", 9: "TMEM allocated", 10: "front kernel's results visible",
         11: "producer knows the unit count", 12: "first complete stage", 13: "first down-projection stage",
         14: "last gate_up stage", 15: "last CTA finished its roles", 16: "last TMEM freed"}


def main(batches):
    import torch

    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    from sm120_moe_bench_b200._lib import LIB_PATH
    raw = C.CDLL(str(LIB_PATH))
    if not hasattr(raw, "vmoe_debug_set_timeline"):
        raise SystemExit("libvmoe.so was built without VMOE_TIMELINE=1: no marks to read")
    dev = torch.device("cuda", 0)
    cfg = synth.CONFIG_LARGE
    layer = synth.make_layer(cfg, seed=0, device=dev)
    routed = ops.MoEWeights(*layer["routed"]).prepare()
    shared = ops.MoEWeights(*layer["shared"]).prepare()
    marks = torch.zeros(32, dtype=torch.int64, device=dev)
    raw.vmoe_debug_set_timeline.argtypes = [C.c_void_p]
    raw.vmoe_debug_set_timeline(marks.data_ptr())
    for M in batches:
        ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2), dev)
        sets = [synth.make_inputs(cfg, M, seed=10 * M + i, device=dev) for i in range(6)]
        out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)
        for i in range(4):
            vm.fused_moe(sets[i][0], routed, ws, router_logits=sets[i][1], shared=shared, out=out)
        torch.cuda.synchronize()
        for rep in (4, 5):
            marks.zero_()
            marks[8:14] = 2 ** 62                      # the "earliest" marks are taken with atomicMin
            torch.cuda.synchronize()
            torch.cuda._sleep(2_000_000)               # both kernels are queued before the GPU reaches them
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            vm.fused_moe(sets[rep][0], routed, ws, router_logits=sets[rep][1], shared=shared, out=out)
            e1.record()
            torch.cuda.synchronize()
            t = marks.cpu().tolist()
            t0 = min(x for x in t[8:14])
            print(f"batch {M}, step {rep - 3}: {e0.elapsed_time(e1) * 1e3:.1f} us between events; " +
                  "; ".join(f"{NAMES[k]} {(t[k] - t0) / 1e3:.1f}" for k in sorted(NAMES) if 0 < t[k] < 2 ** 61))


if __name__ == "__main__":
    main([int(a) for a in sys.argv[1:]] or [1, 2, 4, 8])
