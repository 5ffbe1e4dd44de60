"""Two-GPU tensor-parallel decode step against the single-process CPU restatement (needs two CUDA devices)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, results):
    import torch.distributed as dist

    from singe_b200.llama import LlamaDecoder, Shard
    from tests.llama_util import MEDIUM, make_context, make_weights

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    config = MEDIUM
    context = [40, 0, 129, 700]
    weights = make_weights(config)
    decoder = LlamaDecoder(config, len(context), 768, shard=Shard(rank, world, dist), weights=weights)
    keys, values = make_context(config, decoder.table.page_count())
    gs = slice(rank * decoder.kv_heads, (rank + 1) * decoder.kv_heads)
    for layer in range(config.layers):
        decoder.key_caches[layer].copy_(torch.from_numpy(np.ascontiguousarray(keys[layer][:, :, gs])).to(torch.bfloat16))
        decoder.value_caches[layer].copy_(
            torch.from_numpy(np.ascontiguousarray(values[layer][:, :, gs])).to(torch.bfloat16))
    decoder.table.place_prompts(context)
    rng = np.random.default_rng(11)
    logits, tokens_out = [], []
    for _ in range(2):
        tokens = rng.integers(0, config.vocab, size=len(context))
        next_tokens = decoder.step(tokens)
        torch.cuda.synchronize()
        gathered = [torch.empty_like(decoder.logits) for _ in range(world)]
        dist.all_gather(gathered, decoder.logits)
        logits.append(torch.cat(gathered, dim=1).float().cpu().numpy())
        tokens_out.append(next_tokens.cpu().numpy())
    if rank == 0:
        results["logits"] = logits
        results["tokens"] = tokens_out
        results["status"] = int(decoder.status.item())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_decode_step_matches_the_reference_path():
    import torch.multiprocessing as mp

    from oracle import llama_ref
    from singe_b200.llama import PageTable, rotary_tables
    from tests.gpu_util import BF16_ABS, BF16_REL
    from tests.llama_util import MEDIUM, make_context, make_weights

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, _free_port(), results), nprocs=2, join=True)
    config = MEDIUM
    context = [40, 0, 129, 700]
    weights = make_weights(config)
    table = PageTable.create(len(context), 768, config.page_size)
    keys, values = make_context(config, table.page_count())
    table.place_prompts(context)
    cos, sin = rotary_tables(config.head_dim, config.theta, 768)
    rng = np.random.default_rng(11)
    assert results["status"] == 0
    for index in range(2):
        tokens = rng.integers(0, config.vocab, size=len(context))
        step = table.step([[int(t)] for t in tokens])
        expect = llama_ref.decode_step(config, weights, keys, values, step, cos, sin)
        got = results["logits"][index]
        error = np.abs(got - expect)
        # one more bf16 rounding than the single-GPU path: the partial sums are rounded before the all-reduce
        assert (error <= 2 * BF16_ABS + 2 * BF16_REL * np.abs(expect)).all(), f"max abs err {error.max():.3e}"
        top = np.sort(expect, axis=1)[:, -2:]
        clear = (top[:, 1] - top[:, 0]) > 0.1
        assert (results["tokens"][index][clear] == expect.argmax(axis=1)[clear]).all()
