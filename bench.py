#!/usr/bin/env python3
"""Benchmark of the fused NVFP4 MoE expert layer (decode, large-MoE shape).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--impl ours|reference]

One "step" is one pass of the layer over one batch of M synthetic tokens (hidden 4096, 512 routed
experts top-10 + 1 shared expert, intermediate 1024, NVFP4 weights from seed 0).  Prints ONE JSON
line (rank 0).  ``value`` is tokens/s with inputs resident in HBM, timed with CUDA events;
``e2e`` is the same metric through the operator class with host (pinned) buffers, host<->device
copies inside the timed region; ``roofline`` is the gate_up kernel's algorithmic bytes over its
own event-timed launch duration against the measured HBM copy bandwidth; ``cpu_baseline`` is the
CPU oracle (torch dequantise-then-matmul, all host threads) timed on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("VMOE_NO_VLLM", "1")   # the operator classes do not need the framework to run

METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=64, help="decode batch per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rotate", type=int, default=4, help="distinct input sets cycled through")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-tokens", type=int, default=8)
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "stack"],
                    help="decode: BASELINE config 2 (default, the headline); prefill: config 3 (8192 tokens, "
                         "FP4 TFLOP/s); stack: config 5 shape on one GPU (15 layers, batch 32, CUDA graph)")
    ap.add_argument("--zipf", type=float, default=None, help="prefill: Zipf exponent of the routing bias (1.2 = skewed variant)")
    ap.add_argument("--layers", type=int, default=15)
    ap.add_argument("--path", default="tc", choices=["tc", "gemv"],
                    help="tc: tcgen05 block-scaled path (default); gemv: CUDA-core streaming GEMV path")
    return ap.parse_args()


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle (torch dequantise-then-matmul restatement of the reference's check,
# fused-moe/test_verdict_moe_ext.py:196-218) on a bounded sample of the workload.
# ---------------------------------------------------------------------------------------------
def cpu_sample_problem(tokens: int, seed: int):
    """A bounded sample of the decode workload, built on the CPU: ``tokens`` tokens of the batch with
    only the experts they touch materialised (ids remapped to a dense range)."""
    import numpy as np
    import torch
    from oracle import moe as omoe
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_LARGE
    hidden, logits = synth.make_inputs(cfg, tokens, seed=seed)
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    used, dense = np.unique(ids, return_inverse=True)
    gen = torch.Generator().manual_seed(seed)
    routed = synth.make_expert_weights(len(used), cfg.hidden, cfg.inter, gen, "cpu")
    shared = synth.make_expert_weights(1, cfg.hidden, cfg.inter, gen, "cpu")
    conv = lambda six: omoe.ExpertWeights(*[t.numpy() for t in six])
    return hidden.float().numpy(), dense.reshape(ids.shape).astype(np.int32), w, conv(routed), conv(shared), len(used)


def cpu_time_once(problem):
    from oracle import moe as omoe
    hidden, ids, w, routed, shared, _ = problem
    t0 = time.perf_counter()
    omoe.moe_layer(hidden, ids, w, routed, shared, accum="f32")
    return time.perf_counter() - t0


def cpu_reference():
    """(time_once, kind, threads, description) of the CPU arm: the reference's own host C++ path when its compiled
    library is present (``oracle/_ref``, built by ``oracle/build_ref.py`` where the reference checkout exists:
    quantize_to_nvfp4_e4m3 + host_quantized_reference_single of fused-moe/csrc/verdict_fused_independent.cu, one
    expert per worker thread), otherwise the vectorised restatement in ``oracle/`` on all torch threads."""
    import numpy as np
    from oracle import ref_host
    ref = ref_host.load()
    cores = os.cpu_count() or 1
    if ref is None or ref.hidden != 4096:
        return cpu_time_once, "port", cores, "the CPU oracle (vectorised restatement, torch CPU matmuls)"
    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(max_workers=cores)

    def time_once(problem):
        hidden, ids, w, routed, shared, _ = problem
        t0 = time.perf_counter()
        for m in range(hidden.shape[0]):
            xp, xs = ref.quantize(hidden[m])
            jobs = [(routed, int(e), float(wt)) for e, wt in zip(ids[m], w[m])] + [(shared, 0, 1.0)]
            outs = list(pool.map(lambda j: ref.layer_single(xp, xs, j[0].w13, j[0].w13_sf, j[0].w2, j[0].w2_sf,
                                                            [j[1]], [j[2]]), jobs))
            acc = np.zeros(ref.hidden, np.float32)
            for o in outs:
                acc += o
        return time.perf_counter() - t0

    return (time_once, "reference", min(cores, 11),
            "the reference's compiled host C++ path (host_quantized_reference_single, one expert per thread; "
            "it applies no global scales)")


def run_reference_arm(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    time_once, kind, cores, what = cpu_reference()
    sample_tokens = 1
    problem = cpu_sample_problem(sample_tokens, seed=0)
    for _ in range(max(args.warmup, 0)):
        time_once(problem)
    times = [time_once(problem) for _ in range(max(args.steps, 1))]
    total = sum(times)
    value = sample_tokens * len(times) / total
    sample = (f"{sample_tokens} token(s) of the {args.tokens}-token decode batch per step, "
              f"{problem[5]} routed experts + 1 shared per step, through {what}")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32",
        "data": "synthetic",
        "config": workload_config(args.tokens, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(tokens, gpus):
    return {"workload": "single-GPU decode MoE layer, large-MoE shape (BASELINE config 2)" if gpus == 1 else
            f"decode MoE layer, large-MoE shape (BASELINE config 2 layer), expert parallel over {gpus} GPUs",
            "hidden": 4096, "inter": 1024, "experts": 512, "topk": 10, "shared_experts": 1,
            "tokens_per_gpu": tokens, "weights": "NVFP4 (E2M1 + E4M3 per-16 + fp32 global), N(0,0.02), seed 0",
            "parallelism": "single GPU" if gpus == 1 else f"{gpus} independent replicas",
            "l2": "inputs larger than L2: every step streams > 126 MB of expert weights; input sets rotate"}


# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    from sm120_moe_bench_b200.verdict_moe import VerdictMoEMonolithic

    if world > 1 and args.workload == "stack":
        return run_stack_expert_parallel(args, world, rank, local, dev)
    if world > 1:
        return run_expert_parallel(args, world, rank, local, dev)
    if args.workload == "prefill":
        return run_prefill(args, dev)
    if args.workload == "stack":
        return run_stack(args, dev)

    cfg = synth.CONFIG_LARGE
    M = args.tokens
    layer = synth.make_layer(cfg, seed=0, device=dev)
    routed = ops.MoEWeights(*layer["routed"]).prepare()
    shared = ops.MoEWeights(*layer["shared"]).prepare()
    path = 2 if args.path == "tc" else 1
    shape = vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, max(M, 1), has_shared=True, path=path)
    ws = vm.Workspace(shape, dev)
    sets = [synth.make_inputs(cfg, M, seed=100 * rank + i, device=dev, zipf_s=args.zipf) for i in range(max(args.rotate, 1))]
    out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)

    def step(i):
        h, l = sets[i % len(sets)]
        vm.fused_moe(h, routed, ws, router_logits=l, shared=shared, out=out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    status = ws.status()

    # ---- per-kernel durations, same inputs, each stage bracketed by its own events ---------
    stage_ms = {"gate_up": 0.0, "down": 0.0}
    distinct = []
    for i in range(args.steps):
        h, l = sets[i % len(sets)]
        vm.fused_moe(h, routed, ws, router_logits=l, shared=shared, out=out)   # fills every intermediate table
        ids = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
        w = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
        # A device-side delay goes first so that the host has enqueued every launch and event below before
        # the GPU reaches them: the event intervals then hold kernel time only, no host launch latency.
        torch.cuda._sleep(400_000)
        vm.build_tables(ws, ids, w)                                            # same tables, work queues reset
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        ops.run_stage("gate_up", ws, routed, shared, M)
        ev[1].record()
        ops.run_stage("down", ws, routed, shared, M)
        ev[2].record()
        ev[2].synchronize()
        stage_ms["gate_up"] += ev[0].elapsed_time(ev[1])
        stage_ms["down"] += ev[1].elapsed_time(ev[2])
        distinct.append(int(torch.unique(ids).numel()) + 1)
    U = float(np.mean(distinct))
    K, N = cfg.hidden, cfg.inter
    gate_up_bytes = U * (2 * N * K // 2 + 2 * N * K // 16) + M * (K // 2 + K // 16)
    down_bytes = U * (K * N // 2 + K * N // 16)
    layer_bytes = U * routed.nbytes_per_expert() + M * (K * 2 * 2 + cfg.num_experts * 4)
    peak, peak_kind = measured_peak_gbs()
    gu_s = stage_ms["gate_up"] / args.steps * 1e-3
    dn_s = stage_ms["down"] / args.steps * 1e-3
    kname = "tc_gemm_kernel<2> (gate_up, tcgen05)" if path == 2 else "gate_up_kernel (CUDA-core GEMV)"
    roof = {"bound": "hbm", "kernel": kname, "achieved": gate_up_bytes / gu_s / 1e9, "peak": peak,
            "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
            "unit": "GB/s", "frac": gate_up_bytes / gu_s / 1e9 / peak,
            # DRAM bytes per launch: one ncu capture of this kernel at batch 16 read + wrote 1.044x its
            # algorithmic bytes (profiles/tc_gemm_gate_up_down_decode_bs16_ncu.md); traffic grows with the
            # number of distinct experts like the algorithmic bytes do, so that ratio is applied here
            "traffic": (1.044 if path == 2 else 1.048) * gate_up_bytes,
            "algorithmic_bytes_per_launch": gate_up_bytes, "us_per_launch": gu_s * 1e6,
            "distinct_experts_per_step": U,
            "down_kernel": {"achieved": down_bytes / dn_s / 1e9, "frac": down_bytes / dn_s / 1e9 / peak,
                            "us_per_launch": dn_s * 1e6, "algorithmic_bytes_per_launch": down_bytes},
            "layer": {"achieved": layer_bytes / (ms / args.steps * 1e-3) / 1e9,
                      "frac": layer_bytes / (ms / args.steps * 1e-3) / 1e9 / peak,
                      "algorithmic_bytes_per_step": layer_bytes}}

    # ---- end to end through the operator class with host buffers -----------------------------
    class _Q:  # quant-config attributes the class reads (fused-moe/verdict_moe.py:499-503,519-520)
        g1_alphas, g2_alphas = routed.w13_gs, routed.w2_gs
        a1_gscale = torch.ones_like(routed.w13_gs); a2_gscale = torch.ones_like(routed.w2_gs)
        w1_scale, w2_scale = routed.w13_sf, routed.w2_sf

    class _C:
        experts_per_token = cfg.topk
    VerdictMoEMonolithic.kernel_path = path
    op = VerdictMoEMonolithic(_C(), _Q())
    op.set_shared_expert(shared)
    host_sets = [(h.cpu().pin_memory(), l.cpu().pin_memory()) for h, l in sets]
    host_out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16).pin_memory()
    h_dev = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)
    l_dev = torch.empty(M, cfg.num_experts, dtype=torch.float32, device=dev)

    def e2e_enqueue(k):
        hh, lh = host_sets[k]
        h_dev.copy_(hh, non_blocking=True)
        l_dev.copy_(lh, non_blocking=True)
        o = op.apply(h_dev, routed.w13, routed.w2, l_dev, "SILU", cfg.num_experts, None, None, False)
        host_out.copy_(o, non_blocking=True)

    # The user's call sequence (copy in, apply, copy out) is captured once per host input set and replayed as a
    # CUDA graph, as a serving engine does; every replay still performs both copies.  Eager calls if capture fails.
    e2e_mode, graphs = "eager calls", []
    if world == 1:
        try:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for k in range(len(host_sets)):
                    e2e_enqueue(k)
                side.synchronize()
                for k in range(len(host_sets)):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        e2e_enqueue(k)
                    graphs.append(g)
            torch.cuda.synchronize()
            e2e_mode = "one CUDA graph per host input set: H2D copies + operator call + D2H copy"
        except Exception:  # noqa: BLE001
            graphs = []
            torch.cuda.synchronize()

    def e2e_step(i):
        k = i % len(host_sets)
        if graphs:
            graphs[k].replay()
        else:
            e2e_enqueue(k)
        torch.cuda.current_stream().synchronize()     # the caller reads the result every step

    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.steps):
        e2e_step(i)
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)

    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

    line = None
    if rank == 0:
        tokens_total = M * world * args.steps
        launches_per_step = 6 if M * cfg.topk <= 4096 else 10   # route, tables (1 or 5), quantise, gate_up, down, combine
        line = {
            "metric": METRIC, "value": tokens_total / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32",
            "data": "synthetic", "config": dict(workload_config(M, world), kernel_path=args.path),
            "roofline": roof, "clocks": clocks,
            "e2e": {"value": tokens_total / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": M * (cfg.hidden * 2 + cfg.num_experts * 4),
                    "d2h_bytes_per_step": M * cfg.hidden * 2, "ms_per_step": e2e_ms / args.steps, "mode": e2e_mode},
            "gpu_launches": launches_per_step * args.steps,
            "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            torch.set_num_threads(os.cpu_count() or 1)
            time_once, kind, cores, what = cpu_reference()
            problem = cpu_sample_problem(args.cpu_sample_tokens, seed=0)
            dt = time_once(problem)
            line["cpu_baseline"] = {
                "value": args.cpu_sample_tokens / dt, "unit": UNIT, "cores": cores, "kind": kind,
                "sample": f"{args.cpu_sample_tokens} tokens of the batch, {problem[5]} routed experts + 1 shared, "
                          f"one pass through {what} ({dt:.1f} s)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


NOMINAL_FP4_TFLOPS = 9000.0     # dense FP4, B200 data sheet; no measured FP4 figure is provided


def run_prefill(args, dev):
    """BASELINE config 3: 8192 tokens through the same layer on one GPU; FP4 TFLOP/s of the whole layer
    (2 * M * (T + 1) * 3 * K * N flops) and of the two grouped GEMMs, event-timed."""
    import torch

    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.CONFIG_LARGE
    M = args.tokens if args.tokens != 64 else 8192
    layer = synth.make_layer(cfg, seed=0, device=dev)
    routed = ops.MoEWeights(*layer["routed"]).prepare()
    shared = ops.MoEWeights(*layer["shared"]).prepare()
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2), dev)
    sets = [synth.make_inputs(cfg, M, seed=i, device=dev, zipf_s=args.zipf) for i in range(2)]
    out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    for i in range(args.warmup):
        vm.fused_moe(sets[i % 2][0], routed, ws, router_logits=sets[i % 2][1], shared=shared, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        vm.fused_moe(sets[i % 2][0], routed, ws, router_logits=sets[i % 2][1], shared=shared, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    stage_ms = {"gate_up": 0.0, "down": 0.0}
    for i in range(min(args.steps, 10)):
        ids = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
        w = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
        torch.cuda._sleep(400_000)         # lets the host enqueue everything below ahead of the GPU
        vm.build_tables(ws, ids, w)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record(); ops.run_stage("gate_up", ws, routed, shared, M)
        ev[1].record(); ops.run_stage("down", ws, routed, shared, M)
        ev[2].record(); ev[2].synchronize()
        stage_ms["gate_up"] += ev[0].elapsed_time(ev[1]) / min(args.steps, 10)
        stage_ms["down"] += ev[1].elapsed_time(ev[2]) / min(args.steps, 10)
    clocks = sampler.stop()
    K, N, T = cfg.hidden, cfg.inter, cfg.topk
    flops = 2.0 * M * (T + 1) * 3 * K * N
    gu_flops, dn_flops = flops * 2 / 3, flops / 3
    peak_hbm, kind = measured_peak_gbs()
    bytes_alg = (cfg.num_experts + 1) * routed.nbytes_per_expert() + M * K * 4
    line = {"metric": "moe_layer_prefill_fp4_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32", "data": "synthetic",
            "config": {"workload": "single-GPU prefill MoE layer (BASELINE config 3)", "tokens": M, "zipf_s": args.zipf,
                       "hidden": K, "inter": N, "experts": cfg.num_experts, "topk": T, "shared_experts": 1},
            "tokens_per_s": M / (ms * 1e-3),
            "roofline": {"bound": "tensor", "kernel": "pf_kernel<1> (gate_up, tcgen05, 128-token x 256-row items)",
                         "achieved": gu_flops / (stage_ms["gate_up"] * 1e-3) / 1e12, "peak": NOMINAL_FP4_TFLOPS,
                         "peak_source": "nominal dense FP4 (no measured FP4 peak available)", "unit": "TFLOP/s",
                         "frac": gu_flops / (stage_ms["gate_up"] * 1e-3) / 1e12 / NOMINAL_FP4_TFLOPS, "traffic": None,
                         "us_per_launch": stage_ms["gate_up"] * 1e3,
                         "down_kernel": {"achieved": dn_flops / (stage_ms["down"] * 1e-3) / 1e12,
                                         "us_per_launch": stage_ms["down"] * 1e3},
                         "layer_hbm": {"algorithmic_bytes": bytes_alg, "achieved_gbs": bytes_alg / (ms * 1e-3) / 1e9,
                                       "frac_of_hbm_peak": bytes_alg / (ms * 1e-3) / 1e9 / peak_hbm, "peak_source": kind}},
            "clocks": clocks, "device_status": ws.status()}
    print(json.dumps(line), flush=True)


def run_stack(args, dev):
    """BASELINE config 5 shape on one GPU: ``--layers`` consecutive layers with independent seeded weights,
    ``x <- x + moe(x)``, decode batch ``--tokens`` (default 32), replayed from one CUDA graph.  Reports the
    latency of one pass (= per-token latency of the stack) and tokens/s."""
    import torch

    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ops, synth
    cfg = synth.CONFIG_LARGE
    M = args.tokens if args.tokens != 64 else 32
    L = args.layers
    layers = []
    for li in range(L):
        lay = synth.make_layer(cfg, seed=li, device=dev)
        layers.append((ops.MoEWeights(*lay["routed"]).prepare(), ops.MoEWeights(*lay["shared"]).prepare()))
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2), dev)
    x0, _ = synth.make_inputs(cfg, M, seed=0, device=dev)
    logits = [synth.make_inputs(cfg, M, seed=1000 + li, device=dev)[1] for li in range(L)]
    x = x0.clone()
    def one_pass():
        x.copy_(x0)
        for li in range(L):
            # residual add fused into the combine kernel, in place: x <- x + moe(x)
            vm.fused_moe(x, layers[li][0], ws, router_logits=logits[li], shared=layers[li][1], out=x, residual=x)

    one_pass()                                          # warm: tensor maps, attributes
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        one_pass()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            one_pass()
    torch.cuda.synchronize()
    eager_ref = x.clone()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms_graph = e0.elapsed_time(e1) / args.steps
    same = bool(torch.equal(x, eager_ref))
    e0.record()
    for _ in range(args.steps):
        one_pass()
    e1.record()
    torch.cuda.synchronize()
    ms_eager = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    line = {"metric": "moe_stack_latency_ms", "value": ms_graph, "unit": "ms per pass (per-token latency)", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_graph, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32", "data": "synthetic",
            "config": {"workload": "stack of MoE layers, config-2 shape, residual add, one CUDA graph (BASELINE config 5 on one GPU)",
                       "layers": L, "tokens": M},
            "us_per_layer": ms_graph * 1e3 / L, "tokens_per_s": M / (ms_graph * 1e-3),
            "eager_ms_per_pass": ms_eager, "graph_equals_eager": same, "clocks": clocks, "device_status": ws.status()}
    print(json.dumps(line), flush=True)


def run_stack_expert_parallel(args, world, rank, local, dev):
    """BASELINE config 5: ``--layers`` consecutive MoE layers (independent seeded weights, ``x <- x + moe(x)``)
    at a decode batch of 32 tokens over all ranks (``--tokens`` per rank, default 32 / N), experts split over the
    ranks, dispatch and combine as peer-memory kernels.  Reports the latency of one pass = per-token latency,
    device-timed, max over ranks.  Eager launches: the exchange epoch is a kernel argument, so the pass is not
    replayed from a CUDA graph."""
    import torch
    import torch.distributed as dist

    from sm120_moe_bench_b200 import ep, ops, synth
    cfg = synth.CONFIG_LARGE
    M = args.tokens if args.tokens != 64 else max(32 // world, 1)
    L = args.layers
    first, per = ep.expert_partition(cfg.num_experts, world, rank)
    moes = []
    for li in range(L):
        lay = synth.make_layer(cfg, seed=li, device=dev)                  # identical on every rank (same seed)
        mine = ops.MoEWeights(*[t[first:first + per].contiguous() for t in lay["routed"]]).prepare()
        shared = ops.MoEWeights(*lay["shared"]).prepare()
        del lay
        torch.cuda.empty_cache()
        moes.append(ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, mine, shared, max_local_tokens=M))
    x0, _ = synth.make_inputs(cfg, M, seed=100 * rank, device=dev)
    logits = [synth.make_inputs(cfg, M, seed=1000 + 100 * rank + li, device=dev)[1] for li in range(L)]
    x = x0.clone()
    y = torch.empty_like(x)

    def one_pass():
        x.copy_(x0)
        for li in range(L):
            moes[li].forward(x, logits[li], out=y)
            x.add_(y)                                   # residual

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        one_pass()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        one_pass()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    status = max(m.status() for m in moes)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms, float(status)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t[0].item()
        line = {"metric": "moe_stack_latency_ms", "value": ms, "unit": "ms per pass (per-token latency)", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32", "data": "synthetic",
                "config": {"workload": f"stack of MoE layers, config-2 shape, residual add, expert parallel over {world} GPUs "
                                       "(BASELINE config 5), eager launches",
                           "layers": L, "tokens_per_gpu": M, "tokens": M * world, "experts_per_gpu": per},
                "us_per_layer": ms * 1e3 / L, "tokens_per_s": M * world / (ms * 1e-3), "clocks": clocks,
                "device_status": int(t[1].item())}
        print(json.dumps(line), flush=True)
    for m in moes:
        m.close()
    dist.destroy_process_group()


def run_expert_parallel(args, world, rank, local, dev):
    """N > 1: the same layer with its 512 experts split evenly over the ranks (64 per GPU at N = 8),
    every rank bringing ``--tokens`` tokens of its own (weak scaling); dispatch and combine run as
    peer-memory kernels over NVLink, NCCL is only used for set-up and for the timing barriers."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from sm120_moe_bench_b200 import ep, ops, synth

    cfg = synth.CONFIG_LARGE
    M = args.tokens
    layer = synth.make_layer(cfg, seed=0, device=dev)              # identical on every rank (same seed)
    first, per = ep.expert_partition(cfg.num_experts, world, rank)
    mine = ops.MoEWeights(*[t[first:first + per].contiguous() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*layer["shared"]).prepare()
    del layer
    torch.cuda.empty_cache()
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, mine, shared, max_local_tokens=max(M, 1))
    sets = [synth.make_inputs(cfg, M, seed=100 * rank + i, device=dev) for i in range(max(args.rotate, 1))]
    out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # untimed: how many distinct local experts each input set touches on this rank, and the NVLink rows
    from sm120_moe_bench_b200 import route as dev_route
    local_experts, remote_pairs = [], []
    for h, l in sets:
        ids, _ = dev_route(l, cfg.topk)
        gathered = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        allids = torch.cat(gathered).flatten()
        mine_mask = (allids >= first) & (allids < first + per)
        local_experts.append(int(torch.unique(allids[mine_mask]).numel()) + 1)
        remote_pairs.append(int(((ids.flatten() < first) | (ids.flatten() >= first + per)).sum()))

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        moe.forward(*sets[i % len(sets)], out=out)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        moe.forward(*sets[i % len(sets)], out=out)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    status = moe.status()

    host_sets = [(h.cpu().pin_memory(), l.cpu().pin_memory()) for h, l in sets]
    host_out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16).pin_memory()
    h_dev = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)
    l_dev = torch.empty(M, cfg.num_experts, dtype=torch.float32, device=dev)

    def e2e_step(i):
        hh, lh = host_sets[i % len(host_sets)]
        h_dev.copy_(hh, non_blocking=True)
        l_dev.copy_(lh, non_blocking=True)
        moe.forward(h_dev, l_dev, out=out)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.steps):
        e2e_step(i)
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None

    K, N = cfg.hidden, cfg.inter
    per_expert = mine.nbytes_per_expert()
    my_bytes = float(np.mean(local_experts)) * per_expert
    nv_bytes = float(np.mean(remote_pairs)) * (K // 2 + K // 16 + 16 + K * 4)
    t = torch.tensor([ms, e2e_ms, -my_bytes, -nv_bytes], device=dev, dtype=torch.float64)
    tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    ms, e2e_ms = tmax[0].item(), tmax[1].item()
    total_bytes, total_nv = -tsum[2].item(), -tsum[3].item()
    st = torch.tensor([status], device=dev); dist.all_reduce(st, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        step_s = ms / args.steps * 1e-3
        tokens_total = M * world * args.steps
        config = workload_config(M, world)
        config["parallelism"] = f"expert parallel over {world} GPUs ({per} routed experts per GPU, shared expert replicated), dispatch/combine as NVLink peer-memory kernels"
        config["kernel_path"] = "tc"
        config["zipf_s"] = args.zipf
        line = {
            "metric": METRIC, "value": tokens_total / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32",
            "data": "synthetic", "config": config,
            "roofline": {"bound": "hbm", "kernel": "expert-parallel layer (all kernels of one step, per GPU)",
                         "achieved": total_bytes / world / step_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": total_bytes / world / step_s / 1e9 / peak, "traffic": None,
                         "peak_source": peak_kind, "algorithmic_bytes_per_step_all_gpus": total_bytes,
                         "nvlink_bytes_per_step_all_gpus": total_nv,
                         "nvlink_gbs_per_gpu": total_nv / world / step_s / 1e9},
            "clocks": clocks,
            "e2e": {"value": tokens_total / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": M * (cfg.hidden * 2 + cfg.num_experts * 4) * world,
                    "d2h_bytes_per_step": M * cfg.hidden * 2 * world, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": 13 * args.steps * world,   # route, plan, dispatch, gather, tables, permute, gate_up, down, signal, combine (+3 when tables run as phases)
            "device_status": int(st.item()),
        }
        print(json.dumps(line), flush=True)
    barrier()
    moe.close()
    dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
