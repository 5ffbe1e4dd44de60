"""The allocation-free decode entry point against the regular one.

Hosts that cannot let the library allocate -- a runtime that has handed all device memory to its own pool, or
a decode loop that cannot take the device synchronisation of cudaMalloc -- call
``singe_paged_kv_decode_attention_static_bf16``; its split-K scratch is a fixed array inside the library.
This file sorts last on purpose: a run that stops at the first failure has by then run every other test.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import kernel_sys as ks
from singe_b200 import ops, workloads
from tests.gpu_util import BF16_ABS, BF16_REL, dev, dev_u32, host

pytestmark = pytest.mark.gpu


def _enqueue(name, case, q, k, v, out, lens, table):
    return getattr(ks.lib(), name)(
        int(torch.cuda.current_stream().cuda_stream), out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
        lens.data_ptr(), table.data_ptr(), case.batch, case.heads, case.kv_heads, case.head_dim, case.block_size,
        case.physical_blocks, case.block_table_batch_stride, case.scale)


def _call(name, case, q, k, v, out):
    lens, table = dev(case.lens), dev_u32(case.block_table)
    code = _enqueue(name, case, q, k, v, out, lens, table)
    torch.cuda.synchronize()
    return code


def _problem(seed, lens):
    case = workloads.paged_decode_case(seed=seed, lens=lens)
    rng = np.random.default_rng(seed)
    q = workloads.normal_bf16(rng, (case.batch, case.heads, case.head_dim))
    shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
    k, v = workloads.normal_bf16(rng, shape), workloads.normal_bf16(rng, shape)
    return case, q, k, v


def _oracle(case, q, k, v):
    return oracle.paged_kv_decode_attention_f32(
        q, k, v, case.lens, case.block_table, batch=case.batch, heads=case.heads, kv_heads=case.kv_heads,
        head_dim=case.head_dim, block_size=case.block_size,
        block_table_batch_stride=case.block_table_batch_stride, scale=case.scale)


def test_static_scratch_decode_matches_the_regular_entry_point_twice_in_a_row():
    # Two different problems back to back: the second call must not be affected by what the first left in
    # the shared array (different lengths, so different splits hold live partials).
    for seed, lens in ((101, [3000, 130, 16, 4096, 0, 777]), (102, [64, 2048, 1])):
        case = workloads.paged_decode_case(seed=seed, lens=lens)
        rng = np.random.default_rng(seed)
        q = dev(workloads.normal_bf16(rng, (case.batch, case.heads, case.head_dim)), torch.bfloat16)
        shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
        k = dev(workloads.normal_bf16(rng, shape), torch.bfloat16)
        v = dev(workloads.normal_bf16(rng, shape), torch.bfloat16)
        regular = torch.full_like(q, float("nan"))
        static = torch.full_like(q, float("nan"))
        assert _call("singe_paged_kv_decode_attention_bf16", case, q, k, v, regular) == ks.OK
        assert _call("singe_paged_kv_decode_attention_static_bf16", case, q, k, v, static) == ks.OK
        assert ops.take_device_error() == 0
        a, b = host(static), host(regular)
        assert np.isfinite(a).all()
        error = np.abs(a - b)
        assert (error <= BF16_ABS + BF16_REL * np.abs(b)).all(), f"max abs difference {error.max():.3e}"


def test_static_scratch_decode_matches_the_cpu_restatement_of_the_reference():
    case, q, k, v = _problem(103, [1500, 0, 16, 333, 2049])
    out = torch.full((case.batch, case.heads, case.head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert _call("singe_paged_kv_decode_attention_static_bf16", case, dev(q, torch.bfloat16), dev(k, torch.bfloat16),
                 dev(v, torch.bfloat16), out) == ks.OK
    expect = _oracle(case, q, k, v)
    error = np.abs(host(out) - expect)
    assert (error <= BF16_ABS + BF16_REL * np.abs(expect)).all(), f"max abs error {error.max():.3e}"


def test_static_scratch_calls_queued_back_to_back_on_one_stream_do_not_disturb_each_other():
    # Two problems with different lengths and outputs are enqueued one behind the other with no host wait between
    # them (the second call's kernels may become resident while the first call's combine still reads the shared
    # array; nothing of theirs may touch it before the first call has finished), then once more through a replayed
    # CUDA graph captured after that first use outside capture.
    first = _problem(104, [3000, 130, 16, 4096, 0, 777])
    second = _problem(105, [64, 2048, 1, 900, 4000, 12])
    name = "singe_paged_kv_decode_attention_static_bf16"
    device = []
    for case, q, k, v in (first, second):
        device.append((case, dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16),
                       torch.full((case.batch, case.heads, case.head_dim), float("nan"), dtype=torch.bfloat16,
                                  device="cuda"), dev(case.lens), dev_u32(case.block_table)))

    def enqueue_both():
        for case, q, k, v, out, lens, table in device:
            assert _enqueue(name, case, q, k, v, out, lens, table) == ks.OK

    def check(where):
        for (case, q, k, v), entry in zip((first, second), device):
            expect = _oracle(case, q, k, v)
            error = np.abs(host(entry[4]) - expect)
            assert (error <= BF16_ABS + BF16_REL * np.abs(expect)).all(), f"{where}: max abs error {error.max():.3e}"
            entry[4].fill_(float("nan"))

    enqueue_both()
    torch.cuda.synchronize()
    check("eager")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue_both()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    check("graph replay")
    assert ops.take_device_error() == 0


def test_static_scratch_decode_refuses_what_does_not_fit():
    capacity = ks.lib().singe_paged_kv_decode_attention_static_scratch_floats()
    assert capacity == 2 << 20
    # batch * heads * (head_dim + 1) floats per split: 2048 * 32 * 129 > 2 Mi, so even one split cannot fit.
    one = 16  # any non-null pointer: the size check comes before the device is touched
    code = ks.lib().singe_paged_kv_decode_attention_static_bf16(None, one, one, one, one, one, one, 2048, 32, 8, 128,
                                                                16, 64, 4, 0.1)
    assert code == ks.ERR_STATIC_SCRATCH_EXCEEDED
    assert "fixed scratch" in ks.status_string(code)
    # shapes outside the tiled kernel are refused rather than served by an allocating path
    code = ks.lib().singe_paged_kv_decode_attention_static_bf16(None, one, one, one, one, one, one, 2, 8, 4, 96, 16,
                                                                64, 4, 0.1)
    assert code == ks.ERR_UNSUPPORTED_CONFIGURATION
