"""Checkpoint ingestion (per-expert safetensors entries -> stacked operator layout), on CPU.  A synthetic
checkpoint is written in the naming of the reference's loader (fused-moe/ep_moe_poc.py:26-57), read back
and compared bit for bit; the stacked tensors then feed the oracle."""
import json
import os

import numpy as np
import pytest
import torch

os.environ.setdefault("VMOE_NO_VLLM", "1")


def _layer():
    from sm120_moe_bench_b200 import synth
    cfg = synth.CONFIG_TINY
    return cfg, synth.make_layer(synth.LayerConfig("ckpt", cfg.hidden, cfg.inter, cfg.num_experts, cfg.topk, True), seed=3)


@pytest.mark.parametrize("with_index", [True, False])
def test_round_trip_is_bit_exact(tmp_path, with_index):
    from sm120_moe_bench_b200 import checkpoint as ck
    cfg, layer = _layer()
    ck.save_moe_layer(str(tmp_path), 7, layer["routed"], layer["shared"], shards=3)
    if not with_index:
        os.remove(tmp_path / "model.safetensors.index.json")
    got = ck.load_moe_layer(str(tmp_path), 7, cfg.num_experts, shared_prefix=ck.DEFAULT_SHARED_PREFIX)
    for a, b in zip(got["routed"], layer["routed"]):
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    for a, b in zip(got["shared"], layer["shared"]):
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    # one rank's contiguous block of experts (expert parallelism: gpu = e // (E / G))
    half = ck.load_moe_layer(str(tmp_path), 7, cfg.num_experts // 2, first_expert=cfg.num_experts // 2)
    for a, b in zip(half["routed"], layer["routed"]):
        assert torch.equal(a, b[cfg.num_experts // 2:])
    assert half["shared"] is None


def test_loaded_weights_feed_the_oracle(tmp_path):
    from oracle import moe as omoe
    from sm120_moe_bench_b200 import checkpoint as ck
    from sm120_moe_bench_b200 import synth
    cfg, layer = _layer()
    ck.save_moe_layer(str(tmp_path), 0, layer["routed"], layer["shared"])
    got = ck.load_moe_layer(str(tmp_path), 0, cfg.num_experts, shared_prefix=ck.DEFAULT_SHARED_PREFIX)
    hidden, logits = synth.make_inputs(cfg, 3, seed=5)
    ids, w = omoe.route(logits.numpy(), cfg.topk)
    want = omoe.moe_layer(hidden.float().numpy(), ids, w, omoe.ExpertWeights(*[t.numpy() for t in layer["routed"]]),
                          omoe.ExpertWeights(*[t.numpy() for t in layer["shared"]]))
    have = omoe.moe_layer(hidden.float().numpy(), ids, w, omoe.ExpertWeights(*[t.numpy() for t in got["routed"]]),
                          omoe.ExpertWeights(*[t.numpy() for t in got["shared"]]))
    assert np.array_equal(want, have)


def test_errors(tmp_path):
    from safetensors.torch import load_file, save_file
    from sm120_moe_bench_b200 import checkpoint as ck
    cfg, layer = _layer()
    with pytest.raises(FileNotFoundError):
        ck.load_moe_layer(str(tmp_path), 0, 1)
    ck.save_moe_layer(str(tmp_path), 0, layer["routed"], shards=1)
    with pytest.raises(KeyError):
        ck.load_moe_layer(str(tmp_path), 0, cfg.num_experts + 1)                 # expert that is not there
    with pytest.raises(KeyError):
        ck.load_moe_layer(str(tmp_path), 1, 1)                                   # layer that is not there
    # gate / up global scales that differ: refused, or the gate scale when explicitly allowed (as vLLM does)
    path = tmp_path / "model-00001-of-00001.safetensors"
    t = load_file(str(path))
    key = ck.DEFAULT_EXPERT_PREFIX.format(layer=0, expert=0) + ".up_proj.weight_scale_2"
    t[key] = t[key] * 2
    save_file(t, str(path))
    with pytest.raises(ValueError):
        ck.load_moe_layer(str(tmp_path), 0, 1)
    got = ck.load_moe_layer(str(tmp_path), 0, 1, allow_scale_mismatch=True)
    assert torch.equal(got["routed"][2], layer["routed"][2][:1])
    # wrong block-scale shape
    key = ck.DEFAULT_EXPERT_PREFIX.format(layer=0, expert=1) + ".down_proj.weight_scale"
    t[key] = t[key][:, :-1].contiguous()
    save_file(t, str(path))
    with pytest.raises(ValueError):
        ck.load_moe_layer(str(tmp_path), 0, 2, allow_scale_mismatch=True)
    assert json.load(open(tmp_path / "model.safetensors.index.json"))["weight_map"]
