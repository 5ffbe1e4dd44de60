"""Tensor-parallel plan of the decode step, checked with two gloo ranks on the CPU: every rank takes its shard
of the full weights (KV heads, fused q/k/v columns, o_proj rows, gate/up columns, down_proj rows), computes its
partial products with the CPU restatement, and the sum after o_proj and down_proj must rebuild the unsharded
layer (up to bf16 rounding of the partials)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import llama_ref
from singe_b200.llama import Shard, shard_layer_weights
from tests.llama_util import TINY, make_weights


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    config = TINY
    weights = make_weights(config)
    layer = weights["layers"][0]
    shard = Shard(rank, world, dist)
    mine = shard_layer_weights(layer, config, shard)
    d = config.head_dim
    heads, kv_heads, ffn = config.heads // world, config.kv_heads // world, config.ffn // world
    assert mine["wqkv"].shape == ((heads + 2 * kv_heads) * d, config.hidden)
    assert mine["wo"].shape == (config.hidden, heads * d)
    assert mine["w_gate_up"].shape == (2 * ffn, config.hidden)
    assert mine["w_down"].shape == (config.hidden, ffn)
    rng = np.random.default_rng(3)
    x = llama_ref.bf16(rng.standard_normal((5, config.hidden), dtype=np.float32))
    # attention output of this rank's heads stands in for the attention itself (it is head-local)
    attended_full = llama_ref.bf16(rng.standard_normal((5, config.heads * d), dtype=np.float32))
    attended = attended_full[:, rank * heads * d:(rank + 1) * heads * d]
    partial_o = torch.from_numpy(llama_ref.linear(np.ascontiguousarray(attended), np.ascontiguousarray(mine["wo"])))
    dist.all_reduce(partial_o)
    gate_up = llama_ref.linear(x, mine["w_gate_up"])
    act = llama_ref.silu_mul(gate_up[:, :ffn], gate_up[:, ffn:])
    partial_d = torch.from_numpy(llama_ref.linear(act, np.ascontiguousarray(mine["w_down"])))
    dist.all_reduce(partial_d)
    # q/k/v columns of the fused shard are the rank's heads of the full projections
    qkv = llama_ref.linear(x, mine["wqkv"])
    full_q = llama_ref.linear(x, layer["wq"])[:, rank * heads * d:(rank + 1) * heads * d]
    full_k = llama_ref.linear(x, layer["wk"])[:, rank * kv_heads * d:(rank + 1) * kv_heads * d]
    full_v = llama_ref.linear(x, layer["wv"])[:, rank * kv_heads * d:(rank + 1) * kv_heads * d]
    assert np.array_equal(qkv[:, :heads * d], full_q)
    assert np.array_equal(qkv[:, heads * d:(heads + kv_heads) * d], full_k)
    assert np.array_equal(qkv[:, (heads + kv_heads) * d:], full_v)
    if rank == 0:
        full_o = llama_ref.linear(attended_full, layer["wo"])
        full_d = llama_ref.linear(llama_ref.silu_mul(llama_ref.linear(x, layer["gate"]),
                                                     llama_ref.linear(x, layer["up"])), layer["down"])
        results["o"] = float(np.abs(partial_o.numpy() - full_o).max() / (np.abs(full_o).max() + 1e-9))
        results["d"] = float(np.abs(partial_d.numpy() - full_d).max() / (np.abs(full_d).max() + 1e-9))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_rebuilds_the_unsharded_layer():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, _free_port(), results), nprocs=2, join=True)
    # partials are each rounded to bf16 before the sum: relative error of a couple of bf16 ulps
    assert results["o"] < 2e-2 and results["d"] < 2e-2


def test_shards_must_divide_evenly():
    with pytest.raises(ValueError):
        Shard(0, 3).slice(4)
