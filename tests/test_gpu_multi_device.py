"""One process driving two GPUs: the library's per-device state (raised shared-memory limits, SM count, split-K
workspace, error word, fixed scratch array) must be set up on each device it is used on, whichever comes first.
The reference's LocalCommunicatorGroup drives several devices from one process the same way
(singe-nccl/src/local.rs:256-318).  Skips unless two CUDA devices are visible."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops, workloads
from tests.gpu_util import BF16_ABS, BF16_REL, dev, dev_u32, host

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_decode_cache_write_and_linear_on_device_one_first_then_device_zero():
    case = workloads.paged_decode_case(seed=31, batch=3, lens=[700, 16, 1300], max_len=2048)
    rng = np.random.default_rng(31)
    shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
    q = workloads.normal_bf16(rng, (case.batch, case.heads, case.head_dim))
    rows = workloads.normal_bf16(rng, (4200, case.kv_heads, case.head_dim))  # enough rows for the bulk-copy kernel
    pages = rng.integers(0, case.physical_blocks, size=rows.shape[0])
    slots = rng.integers(0, case.block_size, size=rows.shape[0])
    # distinct positions, so the scatter has one answer
    flat = np.unique(pages * case.block_size + slots)
    pages, slots, rows = flat // case.block_size, flat % case.block_size, rows[: flat.size]
    cache_host = np.zeros(shape, dtype=np.float32)
    assert oracle.kv_cache_write(cache_host, rows, pages, slots) == oracle.OK
    expect = oracle.paged_kv_decode_attention_f32(
        q, cache_host, cache_host, case.lens, case.block_table, batch=case.batch, heads=case.heads,
        kv_heads=case.kv_heads, head_dim=case.head_dim, block_size=case.block_size,
        block_table_batch_stride=case.block_table_batch_stride, scale=case.scale)
    x = workloads.normal_bf16(rng, (64, 1024))
    w = workloads.normal_bf16(rng, (512, 1024), std=0.02)
    linear_expect = oracle.linear_bf16_f32(oracle.f32_to_bf16_bits(x), oracle.f32_to_bf16_bits(w), m=64, n=512, k=1024)
    config = ops.PagedKvDecodeAttentionConfig.contiguous(case.batch, case.heads, case.kv_heads, case.head_dim,
                                                         case.block_size, case.physical_blocks,
                                                         case.block_table_batch_stride, case.scale)
    for device in (1, 0):
        with torch.cuda.device(device):
            key_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
            value_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            d_rows = dev(rows, torch.bfloat16)
            ops.kv_cache_write(key_cache, value_cache, d_rows, d_rows, dev(pages.astype(np.int64)),
                               dev(slots.astype(np.int64)), status=status)
            out = torch.empty((case.batch, case.heads, case.head_dim), dtype=torch.bfloat16, device="cuda")
            ops.paged_kv_decode_attention(out, dev(q, torch.bfloat16), key_cache, value_cache, dev(case.lens),
                                          dev_u32(case.block_table), config)
            y = ops.linear(dev(x, torch.bfloat16), dev(w, torch.bfloat16))
            torch.cuda.synchronize()
            assert int(status.item()) == 0 and ops.take_device_error() == 0
            assert np.array_equal(host(key_cache), cache_host), f"cache write on device {device}"
            error = np.abs(host(out) - expect)
            assert (error <= BF16_ABS + BF16_REL * np.abs(expect)).all(), f"decode on device {device}: {error.max():.3e}"
            error = np.abs(host(y) - linear_expect)
            assert (error <= BF16_ABS + BF16_REL * np.abs(linear_expect)).all(), f"linear on device {device}"
