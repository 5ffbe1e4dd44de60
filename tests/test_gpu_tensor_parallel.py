"""Tensor-parallel decode step on 2, 4 and 8 GPUs against the single-process CPU restatement, and the fused
collectives against the rank-ordered sum (each case skips unless that many CUDA devices are visible)."""
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


def _rank(rank, world, port, results, collective):
    import torch.distributed as dist

    from singe_b200.llama import LlamaDecoder, Shard
    from tests.llama_util import MEDIUM, WIDE, make_context, make_weights

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    config = MEDIUM if world == 2 else WIDE
    context = [40, 0, 129, 700]
    weights = make_weights(config)
    decoder = LlamaDecoder(config, len(context), 768, shard=Shard(rank, world, dist), weights=weights,
                           collective=collective)
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
    decoder.close()
    dist.destroy_process_group()


def _reduce_rank(rank, world, port, results, kind):
    """The fused peer-memory collectives (all-reduce + residual add + RMSNorm in one kernel; ``kind`` = one-shot pull
    or two-phase push) against the sum of the gathered partial rows in f32 in rank order, rounded to bf16, followed by
    the separate add + norm kernel -- over several launches (the epoch advances on the device) and through a
    replayed CUDA graph.  With two ranks that sum is what NCCL's all-reduce returns as well, which is checked too."""
    import torch.distributed as dist

    from singe_b200 import kernel_sys as ks
    from singe_b200.peer import PeerAllReduce, TwoPhaseAllReduce

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    lib = ks.lib()
    rows, width, eps = 64, 4096, 1e-5
    two_phase = kind == "twophase"
    if kind == "oneshot":
        peer = PeerAllReduce(dist, rank, world, rows, width)
    else:
        peer = TwoPhaseAllReduce(dist, rank, world, rows, width, replicated=kind == "pushall")
    generator = torch.Generator(device="cuda").manual_seed(100 + rank)
    shared = torch.Generator(device="cuda").manual_seed(7)  # the residual stream and the gain are replicated
    weight = (1.0 + 0.05 * torch.randn(width, generator=shared, device="cuda")).to(torch.bfloat16)
    hidden = torch.randn((rows, width), generator=shared, device="cuda").to(torch.bfloat16)
    expect_hidden = hidden.clone()
    normed = torch.empty_like(hidden)
    expect_normed = torch.empty_like(hidden)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = int(torch.cuda.current_stream().cuda_stream)
    # the two-phase form keeps a row of the residual stream on its owner only
    per = (rows + world - 1) // world
    mine = slice(rank * per, min(rows, (rank + 1) * per)) if two_phase else slice(0, rows)
    graph = None
    staged = [torch.empty((rows, width), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    for call in range(8):
        which = call & 1
        partial = (0.5 * torch.randn((rows, width), generator=generator, device="cuda")).to(torch.bfloat16)
        gathered = [torch.empty_like(partial) for _ in range(world)]
        dist.all_gather(gathered, partial)
        total = gathered[0].float()
        for other in gathered[1:]:
            total = total + other.float()
        total = total.to(torch.bfloat16)
        if world == 2:
            reduced = partial.clone()
            dist.all_reduce(reduced)
            assert torch.equal(reduced, total)
        assert lib.singe_add_rms_norm_bf16(stream, expect_hidden.data_ptr(), total.data_ptr(),
                                           expect_normed.data_ptr(), weight.data_ptr(), rows, width, eps) == ks.OK
        staged[which].copy_(partial)
        if call < 4:
            # eager: copy the partial rows into the partial buffer (stands for the GEMM), then the fused kernel
            torch.cuda.current_stream().synchronize()
            ctypes_copy(peer.partial_pointer(which), staged[which])
            peer.reduce_add_norm(stream, which, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(), eps,
                                 status.data_ptr())
        else:
            if graph is None:
                # one graph = both collectives back to back, as a layer issues them
                torch.cuda.synchronize()
                dist.barrier()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    s = int(torch.cuda.current_stream().cuda_stream)
                    ctypes_copy(peer.partial_pointer(0), staged[0], s)
                    peer.reduce_add_norm(s, 0, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(), eps,
                                         status.data_ptr())
                    ctypes_copy(peer.partial_pointer(1), staged[1], s)
                    peer.reduce_add_norm(s, 1, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(), eps,
                                         status.data_ptr())
            if which == 0:
                continue  # the graph runs on the odd call, when both staged partials are set
            graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        assert int(status.item()) == 0
        assert torch.equal(hidden[mine], expect_hidden[mine]), f"hidden differs at call {call}"
        assert torch.equal(normed, expect_normed), f"normed differs at call {call}"
    if rank == 0:
        results["reduce_ok"] = True
    dist.barrier()
    peer.close()
    dist.destroy_process_group()


def ctypes_copy(target_pointer, source, stream=None):
    """Device-to-device copy into a raw pointer (the peer buffers are not torch tensors)."""
    from cuda.bindings import runtime as cudart

    if stream is None:
        stream = int(torch.cuda.current_stream().cuda_stream)
    (error,) = cudart.cudaMemcpyAsync(target_pointer, source.data_ptr(), source.numel() * source.element_size(),
                                      cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice, stream)
    assert int(error) == 0


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("kind", ["oneshot", "twophase", "pushall"])
def test_fused_peer_all_reduce_matches_the_rank_ordered_sum_then_norm_bit_for_bit(kind, world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_reduce_rank, args=(world, _free_port(), results, kind), nprocs=world, join=True)
    assert results.get("reduce_ok")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("collective", ["oneshot", "twophase", "pushall", "nccl"])
def test_tensor_parallel_decode_step_matches_the_reference_path(collective, world):
    import torch.multiprocessing as mp

    from oracle import llama_ref
    from singe_b200.llama import PageTable, rotary_tables
    from tests.gpu_util import BF16_ABS, BF16_REL
    from tests.llama_util import MEDIUM, WIDE, make_context, make_weights

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if collective == "nccl" and world > 2:
        pytest.skip("the NCCL path is covered at two ranks")
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(world, _free_port(), results, collective), nprocs=world, join=True)
    config = MEDIUM if world == 2 else WIDE
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
