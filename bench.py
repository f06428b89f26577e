#!/usr/bin/env python3
"""Benchmark of the fused NVFP4 MoE expert layer (hidden 4096, 512 routed experts top-10 + 1 shared expert,
intermediate 1024, NVFP4 weights from seed 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--impl ours|reference] [--workload ...]

One "step" is one pass of the layer over one batch of M synthetic tokens.  Prints ONE JSON line (rank 0).

* ``value``: tokens/s of the 64-token decode batch with inputs resident in HBM, timed with CUDA events.  The timed
  loop of exactly ``--steps`` steps is repeated until at least half a second of device time has passed; the
  median repeat is reported (``repeats``) and the clocks are sampled over all of them.
* ``e2e``: the same metric through the operator class with host (pinned) buffers, host<->device copies inside the
  timed region.
* ``roofline``: the gate_up kernel's algorithmic bytes over its own event-timed launch against the measured HBM
  copy bandwidth; ``sweep``: the same figures for decode batches 1, 4, 16, 64; ``prefill``: 8192 tokens, uniform and
  Zipf(1.2) routing, FP4 TFLOP/s and the HBM fraction beside it.
* ``parity``: three token rows of the timed batch against the CPU oracle (untimed).
* ``cpu_baseline``: the reference's compiled host C++ path (``oracle/_ref``) or, where that library is absent, the
  numpy / torch-CPU restatement (``oracle/``), timed on a bounded sample on this machine's host cores.
* N > 1 (torchrun): the experts are split over the ranks, every rank brings ``--tokens`` tokens, dispatch and
  combine run as NVLink peer-memory kernels; the line carries the bit-identity check against the single-GPU layer
  and the strong-scaling comparison (all tokens on one GPU).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
NOMINAL_FP4_TFLOPS = 9000.0     # dense FP4, B200 data sheet
MIN_TIMED_SECONDS = 0.5
# DRAM bytes per launch of the dominant kernel over its algorithmic bytes, from one ncu capture at batch 16
# (dram__bytes_read.sum + dram__bytes_write.sum); traffic grows with the number of distinct experts like the
# algorithmic bytes do, so the ratio is applied to other batch sizes.  An estimate, labelled as such in the line.
TRAFFIC_RATIO = {"tc": 1.02, "gemv": 1.048}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=64, help="decode batch per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rotate", type=int, default=4, help="distinct input sets cycled through")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="decode: skip the batch sweep and the prefill sub-records")
    ap.add_argument("--cpu-sample-tokens", type=int, default=8)
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "stack"],
                    help="decode: BASELINE config 2 (default, the headline); prefill: config 3 (8192 tokens, "
                         "FP4 TFLOP/s); stack: config 5 (15 layers, batch 32, one CUDA graph per rank)")
    ap.add_argument("--zipf", type=float, default=None, help="Zipf exponent of the routing bias (1.2 = skewed variant)")
    ap.add_argument("--mtp-corr", type=float, default=0.0,
                    help="expert parallel: groups of 6 tokens are the positions of one sequence and share this "
                         "fraction of their logits (0.98 gives the reference's ~71 %% adjacent-token expert reuse)")
    ap.add_argument("--layers", type=int, default=15)
    ap.add_argument("--experts", type=int, default=None,
                    help="prefill: number of routed experts (default 512).  8 experts, top-2 makes the grouped GEMM "
                         "compute-bound: the case that shows the tensor pipe at work")
    ap.add_argument("--topk", type=int, default=None, help="prefill: experts per token (default 10)")
    ap.add_argument("--norm", action="store_true",
                    help="stack (one GPU): pre-norm blocks x <- x + moe(rmsnorm(x)); every layer's combine also normalises "
                         "and quantises the next layer's input (vmoe_extras.next_norm_*), which the next layer takes as codes")
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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        pw = [float(r[3]) for r in self.rows if len(r) >= 9 and r[3].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": reasons, "samples": len(sm)}


def timed_repeats(step, steps, barrier, min_seconds=MIN_TIMED_SECONDS, max_repeats=200, agree=None):
    """Runs the loop of exactly ``steps`` steps, bracketed by ``barrier()`` (+ device synchronise) and CUDA events,
    again and again until ``min_seconds`` of device time have passed.  Returns the per-repeat milliseconds.
    ``agree`` (multi-rank): maps this rank's elapsed total to the value every rank uses for the stop decision, so
    that all ranks run the same number of repeats."""
    import torch
    out, total, i = [], 0.0, 0
    while (agree(total) if agree else total) < min_seconds * 1e3 and len(out) < max_repeats:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            step(i)
            i += 1
        e1.record()
        barrier()
        out.append(e0.elapsed_time(e1))
        total += out[-1]
    return out


def timed_repeats_host(step, steps, barrier, min_seconds=MIN_TIMED_SECONDS, max_repeats=200):
    """The same for work that spans several streams: each repeat is bracketed by ``barrier()`` (all streams idle) and
    timed with CUDA events on the default stream, which waits for nothing in flight at that point."""
    import torch
    out, total, i = [], 0.0, 0
    while total < min_seconds * 1e3 and len(out) < max_repeats:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step(i)
            i += 1
        barrier()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
        total += out[-1]
    return out


# ---------------------------------------------------------------------------------------------
# CPU arm: a bounded sample of the decode workload through the reference's host C++ path or the oracle port.
# Built from the oracle's own quantiser, so this arm never loads the CUDA library.
# ---------------------------------------------------------------------------------------------
def cpu_sample_problem(tokens: int, seed: int):
    """``tokens`` tokens of a decode batch with only the experts they touch materialised (ids remapped to a dense
    range).  Same shapes and value distributions as the device workload: weights N(0, 0.02) -> NVFP4 with one fp32
    global scale per expert matrix, activations bf16 N(0, 1), router logits N(0, 1)."""
    import numpy as np
    import torch
    from oracle import moe as omoe
    from oracle import nvfp4
    K, N, E, T = 4096, 1024, 512, 10
    gen = torch.Generator().manual_seed(seed + 1000003)
    hidden = torch.randn(tokens, K, generator=gen).to(torch.bfloat16).float().numpy()
    logits = torch.randn(tokens, E, generator=gen).numpy()
    ids, w = omoe.route(logits, T)
    used, dense = np.unique(ids, return_inverse=True)

    def experts(n):
        parts = [[] for _ in range(6)]
        for _ in range(n):
            w13 = (torch.randn(2 * N, K, generator=gen) * 0.02).numpy()
            p, s, g = nvfp4.quantize_weight(w13)
            parts[0].append(p); parts[1].append(s); parts[2].append(g)
            w2 = (torch.randn(K, N, generator=gen) * 0.02).numpy()
            p, s, g = nvfp4.quantize_weight(w2)
            parts[3].append(p); parts[4].append(s); parts[5].append(g)
        return omoe.ExpertWeights(*[np.stack(x) if i not in (2, 5) else np.asarray(x, np.float32) for i, x in enumerate(parts)])

    return hidden, dense.reshape(ids.shape).astype(np.int32), w, experts(len(used)), experts(1), len(used)


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
    sample = (f"each step = {sample_tokens} token of the {args.tokens}-token decode batch "
              f"({problem[5]} routed experts + 1 shared), through {what}")
    config = workload_config(args.tokens, args.gpus, args.zipf, args.mtp_corr)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32",
        "data": "synthetic",
        "config": config, "tokens_timed_per_step": sample_tokens,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(tokens, gpus, zipf=None, mtp_corr=0.0):
    """What names the workload -- the same dict from both arms (this build and ``--impl reference``); what names an
    implementation (kernel path, measured reuse) is kept out of it."""
    per = 512 // max(gpus, 1)
    c = {"workload": "single-GPU decode MoE layer, large-MoE shape (BASELINE config 2)" if gpus == 1 else
                     f"decode MoE layer, large-MoE shape (BASELINE config 2 layer), expert parallel over {gpus} GPUs",
         "hidden": 4096, "inter": 1024, "experts": 512, "topk": 10, "shared_experts": 1,
         "tokens_per_gpu": tokens, "weights": "NVFP4 (E2M1 + E4M3 per-16 + fp32 global), N(0,0.02), seed 0",
         "parallelism": "single GPU" if gpus == 1 else
                        f"expert parallel over {gpus} GPUs ({per} routed experts per GPU, shared expert replicated)",
         "l2": "inputs larger than L2: every step streams > 126 MB of expert weights; input sets rotate"}
    if zipf is not None:
        c["zipf_s"] = zipf
    if mtp_corr > 0 and tokens % 6 == 0:
        c["mtp"] = {"positions_per_sequence": 6, "logit_correlation": mtp_corr}
    return c


# ---------------------------------------------------------------------------------------------
# single GPU
# ---------------------------------------------------------------------------------------------
class DecodeBench:
    """The config-2 layer on one GPU: weights once, one workspace and a few rotating input sets per batch size."""

    def __init__(self, dev, path: str, experts: int | None = None, topk: int | None = None):
        import sm120_moe_bench_b200 as vm
        from sm120_moe_bench_b200 import ops, synth
        self.vm, self.ops, self.synth, self.dev = vm, ops, synth, dev
        self.cfg = synth.CONFIG_LARGE
        if experts or topk:         # same hidden / intermediate sizes, fewer experts: the compute-bound variant
            self.cfg = synth.LayerConfig("few-experts", 4096, 1024, experts or 512, topk or 10, True)
        self.layer = synth.make_layer(self.cfg, seed=0, device=dev)
        self.routed = ops.MoEWeights(*self.layer["routed"]).prepare()
        self.shared = ops.MoEWeights(*self.layer["shared"]).prepare()
        self.path_name = path
        self.path = 2 if path == "tc" else 1
        self.peak, self.peak_kind = measured_peak_gbs()

    def case(self, M, steps, warmup, rotate, seed0=0, zipf=None, stage_steps=None, mtp_corr=0.0):
        """Times the layer (and its two GEMM kernels alone) at batch M.  Returns a dict of figures."""
        import numpy as np
        import torch
        vm, ops, cfg = self.vm, self.ops, self.cfg
        ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, max(M, 1), has_shared=True, path=self.path), self.dev)
        group = 6 if (mtp_corr > 0 and M % 6 == 0) else None      # 1 verified + 5 draft positions per sequence
        sets = [self.synth.make_inputs(cfg, M, seed=seed0 + i, device=self.dev, zipf_s=zipf, mtp_group=group, mtp_corr=mtp_corr if group else 0.0)
                for i in range(max(rotate, 1))]
        out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=self.dev)

        def step(i):
            h, l = sets[i % len(sets)]
            vm.fused_moe(h, self.routed, ws, router_logits=l, shared=self.shared, out=out)

        # Each step is replayed from a CUDA graph (one per input set, captured once): at small batches a step is a
        # few tens of microseconds of device time, less than the host needs to issue its launches one by one.
        eager_step, graphs = step, []
        try:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for k in range(len(sets)):
                    eager_step(k)
                side.synchronize()
                for k in range(len(sets)):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        eager_step(k)
                    graphs.append(g)
            torch.cuda.synchronize()
            step = lambda i: graphs[i % len(graphs)].replay()
        except Exception:  # noqa: BLE001
            graphs = []
            torch.cuda.synchronize()
        sampler = ClockSampler(self.dev.index or 0).start()
        for i in range(max(warmup, 3)):
            step(i)
        torch.cuda.synchronize()
        reps = timed_repeats(step, steps, torch.cuda.synchronize)
        ms_step = statistics.median(reps) / steps
        status = ws.status()
        # per-kernel durations: same inputs, each stage bracketed by its own events.  A device-side delay goes first
        # so that the host has enqueued every launch and event before the GPU reaches them: the intervals then hold
        # kernel time only, no host launch latency.
        n = stage_steps or min(steps, 40)
        gu, dn, ex, distinct = [], [], [], []
        for i in range(n):
            h, l = sets[i % len(sets)]
            vm.fused_moe(h, self.routed, ws, router_logits=l, shared=self.shared, out=out)   # fills every table
            ids = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
            w = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
            torch.cuda._sleep(400_000)
            vm.build_tables(ws, ids, w)                                            # same tables, work queue reset
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            ops.run_stage("gate_up", ws, self.routed, self.shared, M)
            ev[1].record()
            ops.run_stage("down", ws, self.routed, self.shared, M)
            ev[2].record()
            ev[2].synchronize()
            gu.append(ev[0].elapsed_time(ev[1])); dn.append(ev[1].elapsed_time(ev[2]))
            distinct.append(int(torch.unique(ids).numel()) + 1)
            if self.path == 2:                         # both projections in the forward's own launch(es)
                torch.cuda._sleep(400_000)
                vm.build_tables(ws, ids, w)
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ev[0].record()
                ops.run_stage("experts", ws, self.routed, self.shared, M)
                ev[1].record()
                ev[1].synchronize()
                ex.append(ev[0].elapsed_time(ev[1]))
        clocks = sampler.stop()
        U = float(np.mean(distinct))
        K, N = cfg.hidden, cfg.inter
        gate_up_bytes = U * (2 * N * K // 2 + 2 * N * K // 16) + M * (K // 2 + K // 16)
        down_bytes = U * (K * N // 2 + K * N // 16)
        layer_bytes = U * self.routed.nbytes_per_expert() + M * (K * 2 * 2 + cfg.num_experts * 4)
        gu_s, dn_s = statistics.median(gu) * 1e-3, statistics.median(dn) * 1e-3
        ex_s = statistics.median(ex) * 1e-3 if ex else gu_s + dn_s
        experts_bytes = gate_up_bytes + down_bytes        # the intermediate's round trip is implementation traffic, not counted
        return {"tokens": M, "ms_per_step": ms_step, "tokens_per_s": M / (ms_step * 1e-3), "repeats": len(reps),
                "launch": "one CUDA graph replay per step" if graphs else "eager launches",
                "distinct_experts_per_step": U,
                "layer_frac": layer_bytes / (ms_step * 1e-3) / 1e9 / self.peak, "layer_gbs": layer_bytes / (ms_step * 1e-3) / 1e9,
                "layer_bytes": layer_bytes,
                "gate_up_us": gu_s * 1e6, "gate_up_frac": gate_up_bytes / gu_s / 1e9 / self.peak, "gate_up_bytes": gate_up_bytes,
                "down_us": dn_s * 1e6, "down_frac": down_bytes / dn_s / 1e9 / self.peak, "down_bytes": down_bytes,
                "experts_us": ex_s * 1e6, "experts_frac": experts_bytes / ex_s / 1e9 / self.peak, "experts_bytes": experts_bytes,
                "clocks": clocks, "device_status": status, "_ws": ws, "_sets": sets, "_out": out}

    def parity_rows(self, case, rows):
        """Three rows of the timed batch against the CPU oracle (router ids of the whole batch bit for bit)."""
        import numpy as np
        import torch
        from oracle import moe as omoe
        from tests import util
        cfg, vm = self.cfg, self.vm
        ws, (h, l), M = case["_ws"], case["_sets"][0], case["tokens"]
        out = vm.fused_moe(h, self.routed, ws, router_logits=l, shared=self.shared)
        torch.cuda.synchronize()
        ids = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).cpu().numpy()
        wd = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).cpu().numpy()
        ids_ref, _ = omoe.route(l.cpu().numpy(), cfg.topk)
        ow = util.to_oracle_weights(self.layer["routed"], np.unique(ids[rows]))
        osh = util.to_oracle_weights(self.layer["shared"])
        ref = omoe.moe_layer(h[rows].float().cpu().numpy(), ids[rows], wd[rows], ow, osh)
        got = out[rows].float().cpu().numpy()
        c, r = util.cosine(got, ref), util.rel_l2(got, ref)
        ma = float(np.max(np.abs(got - ref))) / max(float(np.max(np.abs(ref))), 1e-30)
        return {"against": "CPU oracle (oracle/moe.py), untimed", "rows": list(rows),
                "router_ids_bit_exact": bool(np.array_equal(ids, ids_ref)),
                "cosine": c, "rel_l2": r, "max_abs_over_max_ref": ma,
                "tolerance": {"cosine_min": util.OUT_COSINE_MIN, "rel_l2_max": util.OUT_REL_L2_MAX,
                              "max_abs_frac": util.OUT_MAX_ABS_FRAC},
                "ok": bool(np.array_equal(ids, ids_ref) and c >= util.OUT_COSINE_MIN and r <= util.OUT_REL_L2_MAX
                           and ma <= util.OUT_MAX_ABS_FRAC)}

    def prefill_case(self, M, steps, warmup, zipf):
        import torch
        vm, ops, cfg = self.vm, self.ops, self.cfg
        ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, M, has_shared=True, path=2), self.dev)
        sets = [self.synth.make_inputs(cfg, M, seed=i, device=self.dev, zipf_s=zipf) for i in range(2)]
        out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=self.dev)

        def step(i):
            vm.fused_moe(sets[i % 2][0], self.routed, ws, router_logits=sets[i % 2][1], shared=self.shared, out=out)

        sampler = ClockSampler(self.dev.index or 0).start()
        for i in range(max(warmup, 3)):
            step(i)
        torch.cuda.synchronize()
        reps = timed_repeats(step, steps, torch.cuda.synchronize)
        ms = statistics.median(reps) / steps
        gu, dn = [], []
        for i in range(6):
            ids = ws.view("topk_ids", torch.int32, M * cfg.topk).view(M, cfg.topk).clone()
            w = ws.view("topk_weights", torch.float32, M * cfg.topk).view(M, cfg.topk).clone()
            torch.cuda._sleep(400_000)         # lets the host enqueue everything below ahead of the GPU
            vm.build_tables(ws, ids, w)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record(); ops.run_stage("gate_up", ws, self.routed, self.shared, M)
            ev[1].record(); ops.run_stage("down", ws, self.routed, self.shared, M)
            ev[2].record(); ev[2].synchronize()
            gu.append(ev[0].elapsed_time(ev[1])); dn.append(ev[1].elapsed_time(ev[2]))
        clocks = sampler.stop()
        K, N, T = cfg.hidden, cfg.inter, cfg.topk
        flops = 2.0 * M * (T + 1) * 3 * K * N
        bytes_alg = (cfg.num_experts + 1) * self.routed.nbytes_per_expert() + M * K * 4
        gu_ms, dn_ms = statistics.median(gu), statistics.median(dn)
        return {"tokens": M, "zipf_s": zipf, "ms_per_step": ms, "repeats": len(reps), "tokens_per_s": M / (ms * 1e-3),
                "tflops": flops / (ms * 1e-3) / 1e12, "frac_of_nominal_fp4": flops / (ms * 1e-3) / 1e12 / NOMINAL_FP4_TFLOPS,
                "hbm_gbs": bytes_alg / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": bytes_alg / (ms * 1e-3) / 1e9 / self.peak,
                "algorithmic_bytes": bytes_alg, "flops": flops,
                "gate_up_us": gu_ms * 1e3, "gate_up_tflops": flops * 2 / 3 / (gu_ms * 1e-3) / 1e12,
                "down_us": dn_ms * 1e3, "down_tflops": flops / 3 / (dn_ms * 1e-3) / 1e12,
                "clocks": clocks, "device_status": ws.status()}


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world > 1 and args.workload == "stack":
        return run_stack_expert_parallel(args, world, rank, local, dev)
    if world > 1:
        return run_expert_parallel(args, world, rank, local, dev)
    if args.workload == "prefill":
        return run_prefill(args, dev)
    if args.workload == "stack":
        return run_stack(args, dev)

    from sm120_moe_bench_b200.verdict_moe import VerdictMoEMonolithic
    b = DecodeBench(dev, args.path)
    cfg, routed, shared = b.cfg, b.routed, b.shared
    M = args.tokens
    main = b.case(M, args.steps, args.warmup, args.rotate, seed0=0, zipf=args.zipf, mtp_corr=args.mtp_corr)
    parity = b.parity_rows(main, [0, M // 2, M - 1] if M >= 3 else list(range(M)))
    if b.path == 2:
        kname, kb, kus, kfrac = ("tc_fused_kernel: gate_up + down items of the step in one launch (tcgen05)",
                                 main["experts_bytes"], main["experts_us"], main["experts_frac"])
    else:
        kname, kb, kus, kfrac = "gate_up_kernel (CUDA-core GEMV)", main["gate_up_bytes"], main["gate_up_us"], main["gate_up_frac"]
    roof = {"bound": "hbm", "kernel": kname, "achieved": kb / (kus * 1e-6) / 1e9, "peak": b.peak,
            "peak_source": (b.peak_kind + " (MEASURED_PEAKS.json hbm_gbs: a copy kernel, read + write; a read-only stream "
                            "may exceed it slightly)") if b.peak_kind == "measured" else "fallback 6650 GB/s",
            "unit": "GB/s", "frac": kfrac,
            "traffic": TRAFFIC_RATIO[args.path] * kb,
            "traffic_source": f"estimated: {TRAFFIC_RATIO[args.path]} x algorithmic bytes, the ratio one ncu capture of this "
                              "kernel showed at batch 16 (dram__bytes_read.sum + dram__bytes_write.sum)",
            "algorithmic_bytes_per_launch": kb, "us_per_launch": kus,
            "distinct_experts_per_step": main["distinct_experts_per_step"],
            "gate_up_items_alone": {"achieved": main["gate_up_bytes"] / (main["gate_up_us"] * 1e-6) / 1e9, "frac": main["gate_up_frac"],
                                    "us_per_launch": main["gate_up_us"], "algorithmic_bytes_per_launch": main["gate_up_bytes"]},
            "down_items_alone": {"achieved": main["down_bytes"] / (main["down_us"] * 1e-6) / 1e9, "frac": main["down_frac"],
                                 "us_per_launch": main["down_us"], "algorithmic_bytes_per_launch": main["down_bytes"]},
            "layer": {"achieved": main["layer_gbs"], "frac": main["layer_frac"],
                      "algorithmic_bytes_per_step": main["layer_bytes"]}}

    # ---- end to end through the operator class with host buffers -----------------------------
    class _Q:  # quant-config attributes the class reads (fused-moe/verdict_moe.py:499-503,519-520)
        g1_alphas, g2_alphas = routed.w13_gs, routed.w2_gs
        a1_gscale = torch.ones_like(routed.w13_gs); a2_gscale = torch.ones_like(routed.w2_gs)
        w1_scale, w2_scale = routed.w13_sf, routed.w2_sf

    class _C:
        experts_per_token = cfg.topk
    VerdictMoEMonolithic.kernel_path = b.path
    sets = main["_sets"]
    host_sets = [(h.cpu().pin_memory(), l.cpu().pin_memory()) for h, l in sets]
    # Two lanes (operator instance, device staging buffers, pinned result buffer, stream) take the steps in turn, as a
    # serving engine double-buffers: step i's copy-in overlaps step i-1's kernels and step i-2's copy-out.  Every
    # step still copies its inputs in from pinned host memory and its result out, and the host waits for a lane's
    # previous result before it reuses the lane.
    LANES = 2

    class Lane:
        def __init__(self):
            self.op = VerdictMoEMonolithic(_C(), _Q())
            self.op.set_shared_expert(shared)
            self.host_out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16).pin_memory()
            self.h_dev = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)
            self.l_dev = torch.empty(M, cfg.num_experts, dtype=torch.float32, device=dev)
            self.stream = torch.cuda.Stream()
            self.done = torch.cuda.Event()
            self.graphs = []

        def enqueue(self, k):
            hh, lh = host_sets[k]
            self.h_dev.copy_(hh, non_blocking=True)
            self.l_dev.copy_(lh, non_blocking=True)
            o = self.op.apply(self.h_dev, routed.w13, routed.w2, self.l_dev, "SILU", cfg.num_experts, None, None, False)
            self.host_out.copy_(o, non_blocking=True)

    lanes = [Lane() for _ in range(LANES)]
    # The user's call sequence (copy in, apply, copy out) is captured once per lane and host input set and replayed as
    # a CUDA graph; every replay performs both copies.  Eager calls if capture fails.
    e2e_mode = "eager calls on two streams"
    try:
        for ln in lanes:
            with torch.cuda.stream(ln.stream):
                for k in range(len(host_sets)):
                    ln.enqueue(k)
                ln.stream.synchronize()
                for k in range(len(host_sets)):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=ln.stream):
                        ln.enqueue(k)
                    ln.graphs.append(g)
        torch.cuda.synchronize()
        e2e_mode = "two lanes (streams) in turn; per lane and host input set one CUDA graph: H2D copies + operator call + D2H copy"
    except Exception:  # noqa: BLE001
        for ln in lanes:
            ln.graphs = []
        torch.cuda.synchronize()

    def e2e_step(i):
        ln = lanes[i % LANES]
        k = i % len(host_sets)
        ln.done.synchronize()                          # the caller has read this lane's previous result
        with torch.cuda.stream(ln.stream):
            if ln.graphs:
                ln.graphs[k].replay()
            else:
                ln.enqueue(k)
            ln.done.record(ln.stream)

    def e2e_barrier():
        for ln in lanes:
            ln.stream.synchronize()
        torch.cuda.synchronize()

    sampler = ClockSampler(local).start()
    for i in range(max(args.warmup, 3)):
        e2e_step(i)
    e2e_barrier()
    e2e_reps = timed_repeats_host(e2e_step, args.steps, e2e_barrier)
    e2e_ms = statistics.median(e2e_reps)
    e2e_clocks = sampler.stop()

    ms = main["ms_per_step"] * args.steps
    front = "one-CTA front" if M <= 32 else "route, tables"
    launches_per_step = {"tc": (2 if M <= 4 else 3 if M <= 32 else 4), "gemv": 6}[args.path]
    line = {
        "metric": METRIC, "value": M * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main["ms_per_step"], "repeats": main["repeats"],
        "timed_seconds": main["repeats"] * ms * 1e-3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32",
        "data": "synthetic", "config": workload_config(M, 1, args.zipf, args.mtp_corr), "kernel_path": args.path,
        "launch": main["launch"],
        "roofline": roof, "clocks": main["clocks"],
        "e2e": {"value": M * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": M * (cfg.hidden * 2 + cfg.num_experts * 4),
                "d2h_bytes_per_step": M * cfg.hidden * 2, "ms_per_step": e2e_ms / args.steps, "mode": e2e_mode,
                "repeats": len(e2e_reps), "clocks": e2e_clocks},
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": f"{launches_per_step} ({front}" + (", permuting quantiser" if M > 4 else "") +
                             ", fused gate_up + down + combine kernel)" if args.path == "tc" else "6",
        "parity": parity,
        "device_status": main["device_status"],
    }
    if not args.no_sweep and args.path == "tc":
        sweep = []
        for bs in (1, 4, 16):
            c = b.case(bs, max(args.steps, 100), args.warmup, max(args.rotate, 8), seed0=1000 * bs)
            sweep.append({k: v for k, v in c.items() if not k.startswith("_")})
        sweep.append({k: v for k, v in main.items() if not k.startswith("_")})
        line["sweep"] = sweep
        del main
        torch.cuda.empty_cache()
        line["prefill"] = [b.prefill_case(8192, 10, 3, None), b.prefill_case(8192, 10, 3, 1.2)]
        lib_peak = library_fp4_gemm_tflops(dev, 8192, 8192, 8192)
        for rec in line["prefill"]:       # a measured dense-FP4 rate beside the nominal one (None: no library FP4 GEMM here)
            rec["library_fp4_gemm_8192_cubed_tflops"] = lib_peak
            rec["frac_of_library_fp4_gemm"] = rec["tflops"] / lib_peak if lib_peak else None
    if not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        time_once, kind, cores, what = cpu_reference()
        problem = cpu_sample_problem(args.cpu_sample_tokens, seed=0)
        dt = time_once(problem)
        line["cpu_baseline"] = {
            "value": args.cpu_sample_tokens / dt, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{args.cpu_sample_tokens} tokens of a decode batch, {problem[5]} routed experts + 1 shared, "
                      f"one pass through {what} ({dt:.1f} s)"}
    print(json.dumps(line), flush=True)


def library_fp4_gemm_tflops(dev, M, N, K, iters=20):
    """Dense NVFP4 GEMM [M, K] x [N, K]^T of the vendor library (``torch._scaled_mm`` -> cuBLASLt), event-timed: the
    measured stand-in for a dense-FP4 peak, which MEASURED_PEAKS.json does not hold.  Random codes, constant block
    scales; None where this torch build has no FP4 GEMM."""
    import torch
    try:
        a = torch.randint(0, 255, (M, K // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
        w = torch.randint(0, 255, (N, K // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)

        def scales(rows):
            return torch.full((((rows + 127) // 128 * 128) * ((K // 16 + 3) // 4 * 4),), 0.5, device=dev).to(torch.float8_e4m3fn)
        sa, sw = scales(M), scales(N)
        call = lambda: torch._scaled_mm(a, w.t(), scale_a=sa, scale_b=sw, out_dtype=torch.bfloat16)
        for _ in range(5):
            call()
        torch.cuda.synchronize()
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                call()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            best = ms if best is None else min(best, ms)
        return 2.0 * M * N * K / (best * 1e-3) / 1e12
    except Exception:
        return None


def run_prefill(args, dev):
    """BASELINE config 3: 8192 tokens through the same layer on one GPU; FP4 TFLOP/s of the whole layer
    (2 * M * (T + 1) * 3 * K * N flops) and of the two grouped GEMMs, event-timed."""
    b = DecodeBench(dev, "tc", args.experts, args.topk)
    M = args.tokens if args.tokens != 64 else 8192
    c = b.prefill_case(M, args.steps, args.warmup, args.zipf)
    cfg = b.cfg
    # measured dense-FP4 references of the vendor library: a large square GEMM (burst peak) and one dense GEMM with the
    # gate_up projection's row count and sizes (all token rows against ONE expert's weights)
    lib_peak = library_fp4_gemm_tflops(dev, 8192, 8192, 8192)
    lib_same = library_fp4_gemm_tflops(dev, M * (cfg.topk + 1), 2 * cfg.inter, cfg.hidden)
    fp4_peak = lib_peak if lib_peak else NOMINAL_FP4_TFLOPS
    line = {"metric": "moe_layer_prefill_fp4_tflops", "value": c["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": c["ms_per_step"], "repeats": c["repeats"],
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32", "data": "synthetic",
            "config": {"workload": "single-GPU prefill MoE layer (BASELINE config 3)" if not (args.experts or args.topk) else
                                   "single-GPU prefill MoE layer, config-3 sizes with fewer experts (compute-bound variant)",
                       "tokens": M, "zipf_s": args.zipf,
                       "hidden": cfg.hidden, "inter": cfg.inter, "experts": cfg.num_experts, "topk": cfg.topk, "shared_experts": 1},
            "tokens_per_s": c["tokens_per_s"],
            "roofline": {"bound": "tensor", "kernel": ("pair_kernel<1> (gate_up, tcgen05 cta_group::2, 256-token x 256-row items on CTA pairs)"
                                                        if int(os.environ.get("VMOE_PF_PAIR", "0") or 0) & 1
                                                        else "pf_kernel<1> (gate_up, tcgen05, 128-token x 256-row items)"),
                         "achieved": c["gate_up_tflops"], "peak": fp4_peak,
                         "peak_source": ("measured in this run: dense NVFP4 GEMM 8192^3 of the vendor library (torch._scaled_mm); "
                                         "MEASURED_PEAKS.json holds no FP4 figure") if lib_peak else
                                        "nominal dense FP4 (MEASURED_PEAKS.json holds no FP4 figure; no library FP4 GEMM in this torch)",
                         "unit": "TFLOP/s", "frac": c["gate_up_tflops"] / fp4_peak, "traffic": None,
                         "nominal_dense_fp4_tflops": NOMINAL_FP4_TFLOPS, "frac_of_nominal": c["gate_up_tflops"] / NOMINAL_FP4_TFLOPS,
                         "library_dense_gemm_same_sizes": {"rows": M * (cfg.topk + 1), "n": 2 * cfg.inter, "k": cfg.hidden, "tflops": lib_same,
                                                           "note": "one dense GEMM of the gate_up projection's total row count against a single "
                                                                   "expert's weights, no SwiGLU / re-quantisation epilogue"},
                         "us_per_launch": c["gate_up_us"],
                         "down_kernel": {"achieved": c["down_tflops"], "us_per_launch": c["down_us"]},
                         "layer_hbm": {"algorithmic_bytes": c["algorithmic_bytes"], "achieved_gbs": c["hbm_gbs"],
                                       "frac_of_hbm_peak": c["frac_of_hbm_peak"], "peak_source": b.peak_kind}},
            "clocks": c["clocks"], "device_status": c["device_status"]}
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

    if args.norm:
        gen = torch.Generator(device=dev).manual_seed(77)
        gammas = [(1.0 + 0.05 * torch.randn(cfg.hidden, generator=gen, device=dev)).float() for _ in range(L)]
        rows = [ops.QuantizedRows(M, cfg.hidden, dev), ops.QuantizedRows(M, cfg.hidden, dev)]

        def one_pass():
            x.copy_(x0)
            ops.rmsnorm_quantize(x, gammas[0], 1e-6, out=rows[0])            # the first block's input
            for li in range(L):
                cur, nxt = rows[li % 2], rows[(li + 1) % 2]
                # x <- x + moe(norm(x)); the same kernel leaves norm(x) for the next block as bf16 rows + FP4 codes
                vm.fused_moe(cur.normed, layers[li][0], ws, router_logits=logits[li], shared=layers[li][1], out=x, residual=x,
                             hidden_quantized=cur, next_norm=(gammas[li + 1], 1e-6) if li + 1 < L else None,
                             next_rows=nxt if li + 1 < L else None)
    else:
        def one_pass():
            x.copy_(x0)
            for li in range(L):
                # residual add fused into the combine, in place: x <- x + moe(x)
                vm.fused_moe(x, layers[li][0], ws, router_logits=logits[li], shared=layers[li][1], out=x, residual=x)

    one_pass()                                          # warm: tensor maps, attributes
    torch.cuda.synchronize()
    eager_ref = x.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        one_pass()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            one_pass()
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index or 0).start()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    reps = timed_repeats(lambda i: graph.replay(), args.steps, torch.cuda.synchronize)
    ms_graph = statistics.median(reps) / args.steps
    same = bool(torch.equal(x, eager_ref))
    ereps = timed_repeats(lambda i: one_pass(), args.steps, torch.cuda.synchronize, min_seconds=0.2)
    ms_eager = statistics.median(ereps) / args.steps
    clocks = sampler.stop()
    line = {"metric": "moe_stack_latency_ms", "value": ms_graph, "unit": "ms per pass (per-token latency)", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_graph, "repeats": len(reps), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32", "data": "synthetic",
            "config": {"workload": "stack of MoE layers, config-2 shape, residual add, one CUDA graph (BASELINE config 5 on one GPU)" +
                                   (", pre-norm blocks with RMSNorm + next-layer quantisation fused behind every combine" if args.norm else ""),
                       "layers": L, "tokens": M},
            "us_per_layer": ms_graph * 1e3 / L, "tokens_per_s": M / (ms_graph * 1e-3),
            "eager_ms_per_pass": ms_eager, "graph_equals_eager": same, "clocks": clocks, "device_status": ws.status()}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# expert parallel (N > 1)
# ---------------------------------------------------------------------------------------------
def run_stack_expert_parallel(args, world, rank, local, dev):
    """BASELINE config 5: ``--layers`` consecutive MoE layers (independent seeded weights, ``x <- x + moe(x)``)
    at a decode batch of 32 tokens over all ranks (``--tokens`` per rank, default 32 / N), experts split over the
    ranks, dispatch and combine as peer-memory kernels, the residual fused into the combine.  One CUDA graph per
    rank holds the whole pass; its replay is checked against the eager pass bit for bit.  Reports the latency of
    one pass = per-token latency, device-timed, max over ranks."""
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

    def one_pass():
        x.copy_(x0)
        for li in range(L):
            moes[li].forward(x, logits[li], out=x, residual=x)      # x <- x + moe(x), fused into the combine

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def agree(total_ms):
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return t.item()

    for _ in range(3):
        one_pass()
    barrier()
    eager_ref = x.clone()
    mode, graph = "eager launches", None
    try:
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            one_pass()
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                one_pass()
        torch.cuda.synchronize()
        graph, mode = g, "one CUDA graph per rank"
    except Exception as exc:  # noqa: BLE001
        mode = f"eager launches (graph capture failed: {type(exc).__name__})"
        torch.cuda.synchronize()
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        graph = None                                    # all ranks replay or none does: they must stay in step
    run = (lambda i: graph.replay()) if graph is not None else (lambda i: one_pass())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(max(args.warmup, 3)):
        run(i)
    barrier()
    same = bool(torch.equal(x, eager_ref))
    reps = timed_repeats(run, args.steps, barrier, agree=agree)
    ms = statistics.median(reps) / args.steps
    status = max(m.status() for m in moes)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms, float(status), 0.0 if same else 1.0], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t[0].item()
        line = {"metric": "moe_stack_latency_ms", "value": ms, "unit": "ms per pass (per-token latency)", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "repeats": len(reps), "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32", "data": "synthetic",
                "config": {"workload": f"stack of MoE layers, config-2 shape, residual add fused into the combine, expert parallel over "
                                       f"{world} GPUs (BASELINE config 5), {mode}",
                           "layers": L, "tokens_per_gpu": M, "tokens": M * world, "experts_per_gpu": per},
                "us_per_layer": ms * 1e3 / L, "tokens_per_s": M * world / (ms * 1e-3), "clocks": clocks,
                "parity": {"graph_replay_equals_eager_on_all_ranks": t[2].item() == 0.0},
                "device_status": int(t[1].item())}
        print(json.dumps(line), flush=True)
    barrier()
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

    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ep, ops, synth
    from sm120_moe_bench_b200 import route as dev_route

    cfg = synth.CONFIG_LARGE
    M = args.tokens
    group = 6 if args.mtp_corr > 0 else None
    layer = synth.make_layer(cfg, seed=0, device=dev)              # identical on every rank (same seed)
    first, per = ep.expert_partition(cfg.num_experts, world, rank)
    mine = ops.MoEWeights(*[t[first:first + per].contiguous() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*layer["shared"]).prepare()
    full = ops.MoEWeights(*layer["routed"]).prepare()
    sets = [synth.make_inputs(cfg, M, seed=100 * rank + i, device=dev, zipf_s=args.zipf, mtp_group=group, mtp_corr=args.mtp_corr)
            for i in range(max(args.rotate, 1))]
    # untimed, before the full layer is released: what ONE GPU holding all experts computes for this rank's tokens
    # (the bit-identity reference) and, on rank 0, how long one GPU takes for the tokens of ALL ranks (strong scaling)
    ws1 = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, max(M, 1), has_shared=True, path=2), dev)
    single = [vm.fused_moe(h, full, ws1, router_logits=l, shared=shared).clone() for h, l in sets] if M else []
    one_gpu_ms = None
    if rank == 0 and M:
        Mall = M * world
        wsA = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, Mall, has_shared=True, path=2), dev)
        allsets = [synth.make_inputs(cfg, Mall, seed=7000 + i, device=dev, zipf_s=args.zipf, mtp_group=group, mtp_corr=args.mtp_corr)
                   for i in range(2)]
        oA = torch.empty(Mall, cfg.hidden, dtype=torch.bfloat16, device=dev)
        stepA = lambda i: vm.fused_moe(allsets[i % 2][0], full, wsA, router_logits=allsets[i % 2][1], shared=shared, out=oA)
        for i in range(5):
            stepA(i)
        torch.cuda.synchronize()
        one_gpu_ms = statistics.median(timed_repeats(stepA, 20, torch.cuda.synchronize, min_seconds=0.2)) / 20
        del wsA, allsets, oA
    del full, ws1, layer
    torch.cuda.empty_cache()
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, mine, shared, max_local_tokens=max(M, 1))
    out = torch.empty(M, cfg.hidden, dtype=torch.bfloat16, device=dev)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def agree(total_ms):
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return t.item()

    # untimed: how many distinct local experts each input set touches on this rank, and the NVLink rows
    local_experts, remote_pairs, reuse = [], [], []
    for h, l in sets:
        ids, _ = dev_route(l, cfg.topk)
        gathered = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        allids = torch.cat(gathered).flatten()
        mine_mask = (allids >= first) & (allids < first + per)
        local_experts.append(int(torch.unique(allids[mine_mask]).numel()) + 1)
        remote_pairs.append(int(((ids.flatten() < first) | (ids.flatten() >= first + per)).sum()))
        if group:
            reuse.append(synth.adjacent_reuse(ids, group))

    def step(i):
        moe.forward(*sets[i % len(sets)], out=out)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    equal, maxdiff = True, 0.0
    for i in range(max(args.warmup, len(sets), 3)):
        step(i)
        if M:
            equal = equal and bool(torch.equal(out, single[i % len(sets)]))     # synchronises; untimed
            maxdiff = max(maxdiff, float((out.float() - single[i % len(sets)].float()).abs().max()))
    barrier()
    reps = timed_repeats(step, args.steps, barrier, agree=agree)
    ms = statistics.median(reps)
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

    for i in range(max(args.warmup, 3)):
        e2e_step(i)
    barrier()
    e2e_ms = statistics.median(timed_repeats(e2e_step, args.steps, barrier, agree=agree))
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
    okr = torch.tensor([1 if equal else 0], device=dev); dist.all_reduce(okr, op=dist.ReduceOp.SUM)
    mdf = torch.tensor([maxdiff], device=dev, dtype=torch.float64); dist.all_reduce(mdf, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        step_s = ms / args.steps * 1e-3
        tokens_total = M * world * args.steps
        config = workload_config(M, world, args.zipf, args.mtp_corr)
        line = {
            "metric": METRIC, "value": tokens_total / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, len(sets), 3), "ms_per_step": ms / args.steps, "repeats": len(reps),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4(w4a4)->f32",
            "data": "synthetic", "config": config, "kernel_path": "tc",
            "exchange": "dispatch/combine as NVLink peer-memory kernels (no NCCL on the data path)",
            "adjacent_expert_reuse": float(np.mean(reuse)) if group else None,
            "roofline": {"bound": "hbm", "kernel": "expert-parallel layer (all kernels of one step, per GPU)",
                         "achieved": total_bytes / world / step_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": total_bytes / world / step_s / 1e9 / peak, "traffic": None,
                         "peak_source": peak_kind, "algorithmic_bytes_per_step_all_gpus": total_bytes,
                         "distinct_local_experts_rank0": float(np.mean(local_experts)),
                         "nvlink_bytes_per_step_all_gpus": total_nv,
                         "nvlink_gbs_per_gpu": total_nv / world / step_s / 1e9},
            "strong_scaling": {"tokens": M * world, "one_gpu_ms_per_step": one_gpu_ms, "n_gpu_ms_per_step": ms / args.steps,
                               "speedup_over_one_gpu": (one_gpu_ms / (ms / args.steps)) if one_gpu_ms else None,
                               "note": "the same total batch through the single-GPU layer on rank 0 (all experts on one GPU), untimed region"},
            "parity": {"ep_vs_single_gpu": "bit-identical" if int(okr.item()) == world else "DIFFERS",
                       "ranks_ok": int(okr.item()), "max_abs_diff": mdf.item(), "checked": "every warm-up step's output against the single-GPU layer's (torch.equal)"},
            "clocks": clocks,
            "e2e": {"value": tokens_total / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": M * (cfg.hidden * 2 + cfg.num_experts * 4) * world,
                    "d2h_bytes_per_step": M * cfg.hidden * 2 * world, "ms_per_step": e2e_ms / args.steps},
            # router, dispatch (+ plan), gather + tables, experts, combine; above the small-batch threshold the
            # received-row permutation, the second expert kernel and the flag kernel are launches of their own
            "gpu_launches": (5 if M * cfg.topk <= min(int(os.environ.get("VMOE_SMALL_PER_EXPERT", "10")), 16) * per else 8)
                            * args.steps * world,
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
