"""The allocation-free decode entry point against the regular one.

Hosts that cannot let the library allocate -- a runtime that has handed all device memory to its own pool, or
a decode loop that cannot take the device synchronisation of cudaMalloc -- call
``singe_paged_kv_decode_attention_static_bf16``; its split-K scratch is a fixed array inside the library.
This file sorts last on purpose: a run that stops at the first failure has by then run every other test.
"""
import numpy as np
import pytest
import torch

from singe_b200 import kernel_sys as ks
from singe_b200 import ops, workloads
from tests.gpu_util import BF16_ABS, BF16_REL, dev, dev_u32, host

pytestmark = pytest.mark.gpu


def _call(name, case, q, k, v, out):
    lens, table = dev(case.lens), dev_u32(case.block_table)
    code = getattr(ks.lib(), name)(
        int(torch.cuda.current_stream().cuda_stream), out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
        lens.data_ptr(), table.data_ptr(), case.batch, case.heads, case.kv_heads, case.head_dim, case.block_size,
        case.physical_blocks, case.block_table_batch_stride, case.scale)
    torch.cuda.synchronize()
    return code


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
