"""Child process of tests/test_gpu_ep.py (one per GPU, started by torchrun): every rank holds a
slice of the experts and its own tokens; its expert-parallel output must equal, bit for bit, what
one GPU holding all experts computes for the same tokens."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import sm120_moe_bench_b200 as vm
    from sm120_moe_bench_b200 import ep, ops, synth

    cfg = synth.LayerConfig("epw", 1024, 512, 32, 4, True)
    layer = synth.make_layer(cfg, seed=7)                       # same seed: every rank draws the same layer
    full = ops.MoEWeights(*[t.cuda() for t in layer["routed"]]).prepare()
    shared = ops.MoEWeights(*[t.cuda() for t in layer["shared"]]).prepare()
    first, per = ep.expert_partition(cfg.num_experts, world, rank)
    mine = ops.MoEWeights(*[t[first:first + per].contiguous().cuda() for t in layer["routed"]]).prepare()
    max_tok = 96
    moe = ep.ExpertParallelMoE(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, mine, shared, max_local_tokens=max_tok)
    ws = vm.Workspace(vm.MoEShape(cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, max_tok, has_shared=True, path=2))
    ok = True
    # ragged and empty batches; 96 tokens take the token-major kernels at every world size
    for it, M in enumerate([96, 40, 7 + rank, 0 if rank == 0 else 3, 33]):
        hidden, logits = synth.make_inputs(cfg, max(M, 1), seed=100 * it + rank)
        hidden, logits = hidden[:M].cuda().contiguous(), logits[:M].cuda().contiguous()
        out = moe.forward(hidden, logits)
        torch.cuda.synchronize()
        st = moe.status()
        if M:
            ref = vm.fused_moe(hidden, full, ws, router_logits=logits, shared=shared)
            same = torch.equal(out, ref)
        else:
            same = True
        if st != 0 or not same:
            ok = False
            print(f"rank {rank} iter {it} M {M}: status {st} equal {same}", flush=True)
    # one captured call, replayed: equal to the eager result, with the residual fused into the combine
    M = 24
    hidden, logits = synth.make_inputs(cfg, M, seed=900 + rank)
    hidden, logits = hidden.cuda(), logits.cuda()
    eager = moe.forward(hidden, logits, residual=hidden).clone()
    ref = hidden + vm.fused_moe(hidden, full, ws, router_logits=logits, shared=shared)
    out = torch.empty_like(hidden)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        moe.forward(hidden, logits, out=out, residual=hidden)
        side.synchronize()
        dist.barrier()
        with torch.cuda.graph(graph, stream=side):
            moe.forward(hidden, logits, out=out, residual=hidden)
    torch.cuda.synchronize()
    dist.barrier()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    if moe.status() != 0 or not torch.equal(out, eager) or not torch.equal(eager, ref):
        ok = False
        print(f"rank {rank}: graph replay differs from eager / single GPU", flush=True)
    dist.barrier()
    moe.close()
    dist.destroy_process_group()
    if ok:
        print("EP_WORKER_OK", flush=True)
    else:
        sys.exit(1)


if __name__ == "__main__":
    main()
