"""Development aid: cycles per warp role of the token-major tensor-core kernels (single CTA and CTA pair).

Needs the library built with the counters compiled in::

    VMOE_PROFILE=1 python sm120_moe_bench_b200/build.py --force
    python -m sm120_moe_bench_b200.role_cycles [--experts E --topk T] [--tokens M]

(an ordinary build has no counters and this module refuses to run).  It runs the 8192-token layer once, then the
gate_up and the down projection alone -- first on the single-CTA kernels, then on the CTA pairs -- and prints per
projection the event-timed launch and, per work item, how long the MMA warp waited for data, waited for the
accumulator and issued, how long the producers waited for a free ring slot, and how long an epilogue warp waited
and worked.  Numbers of one launch on a cold GPU: shares, not sustained rates.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os

os.environ.setdefault("VMOE_NO_VLLM", "1")

SINGLE = ["MMA warp: waiting for a stage", "MMA warp: waiting for the accumulator", "MMA warp: issuing",
          "epilogue warp: waiting", "epilogue warp: working", "producer: waiting for a slot"]
PAIR = {0: "MMA warp: waiting for a stage", 2: "MMA warp: waiting for the accumulator", 3: "MMA warp: issuing",
        4: "producer (even CTA): waiting for a slot", 5: "producer (odd CTA): waiting for a slot",
        6: "epilogue warp: waiting", 7: "epilogue warp: working", 10: "MMA warp: whole loop"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=512)
    ap.add_argument("--topk", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=8192)
    args = ap.parse_args()
    import torch

    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    from sm120_moe_bench_b200._lib import LIB_PATH
    raw = C.CDLL(str(LIB_PATH))
    if not hasattr(raw, "vmoe_debug_read_pair_profile"):
        raise SystemExit("libvmoe.so was built without VMOE_PROFILE=1: no counters to read")
    cfg = synth.LayerConfig("roles", 4096, 1024, args.experts, args.topk, True)
    M = args.tokens
    layer = synth.make_layer(cfg, seed=0, device="cuda")
    routed = ops.MoEWeights(*layer["routed"]).prepare()
    shared = ops.MoEWeights(*layer["shared"]).prepare()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2))
    hidden, logits = synth.make_inputs(cfg, M, seed=1, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for pair in (0, 1):
        os.environ["VMOE_PF_PAIR"] = "3" if pair else "0"          # bit 0: gate_up on pairs, bit 1: down on pairs
        vm.fused_moe(hidden, routed, ws, router_logits=logits, shared=shared)
        torch.cuda.synchronize()
        ids = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
        w = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
        buf = (C.c_ulonglong * 16)()
        read = raw.vmoe_debug_read_pair_profile if pair else raw.vmoe_debug_read_profile
        read(buf)                                        # clears what the whole-layer run counted
        for stage in ("gate_up", "down"):
            vm.build_tables(ws, ids, w)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.run_stage(stage, ws, routed, shared, M)
            e1.record()
            torch.cuda.synchronize()
            read(buf)
            v = list(buf)
            items = v[8] if pair else v[6]
            ctas = sms // 2 if pair else sms
            print(f"{'CTA pairs' if pair else 'single CTA'}, {stage}: {e0.elapsed_time(e1) * 1e3:.0f} us, {items} items "
                  f"({'256' if pair else '128'} tokens x 256 weight rows each) on {ctas} {'pairs' if pair else 'CTAs'}")
            rows = [(PAIR[i], v[i]) for i in sorted(PAIR)] if pair else list(zip(SINGLE, v[:6]))
            for name, x in rows:
                print(f"    {name:42s} {x / max(items, 1):9.0f} cycles per item")


if __name__ == "__main__":
    main()
