"""bf16 linear-layer GEMM on the tcgen05 tensor core against the CPU restatement of the reference GEMM."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops
from singe_b200 import kernel_sys as ks
from tests.gpu_util import assert_close_bf16, dev, host

pytestmark = pytest.mark.gpu


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _case(m, n, k, seed=2):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)            # X ~ N(0, 1)
    w = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)   # W ~ N(0, 0.02)
    return x, w


@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (16, 512, 1024), (128, 384, 64), (200, 136, 72), (256, 256, 4096),
                                   (129, 1000, 520), (64, 4096, 4096), (1, 14336, 4096), (1024, 9728, 128),
                                   (1000, 9736, 136)])
def test_linear_matches_the_oracle_bf16_and_f32(m, n, k):
    # (the last two shapes have at least one 256 x 256 tile per SM: the form with two M sub-tiles per CTA, with and
    # without M, N and K tails)
    x, w = _case(m, n, k)
    y = ops.linear(x, w)
    y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ops.matmul_bf16(y32, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref = oracle.linear_bf16_f32(_bits(x), _bits(w), m=m, n=n, k=k)
    assert_close_bf16(host(y32), ref, f"matmul_bf16_f32 {m}x{n}x{k}")
    assert_close_bf16(host(y), oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(ref)), f"linear bf16 {m}x{n}x{k}")
    # the f32 result is far tighter than the bf16 tolerance: accumulation order is the only difference
    scale = np.abs(ref).max() + 1e-6
    assert np.abs(host(y32) - ref).max() / scale < 2e-3


@pytest.mark.parametrize("m,n,k,splits", [(64, 4096, 4096, 0), (64, 4096, 14336, 0), (64, 4096, 1792, 0),
                                          (64, 4096, 512, 0), (128, 768, 4096, 0), (5, 1000, 520, 4),
                                          (1, 136, 200, 8), (128, 4096, 4096, 2), (33, 264, 4096, 8)])
def test_split_k_over_a_cluster_matches_the_oracle(m, n, k, splits):
    # One M tile and few N tiles: K is split over a thread-block cluster that reduces through distributed shared
    # memory (splits = 0 lets the shape decide; forced values cover N and K tails and splits that get no K at all).
    x, w = _case(m, n, k, seed=5)
    lib = ks.lib()
    assert lib.singe_matmul_set_splits(splits) == ks.OK
    try:
        y = ops.linear(x, w)
        y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
        ops.matmul_bf16(y32, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
        again = torch.empty_like(y32)
        ops.matmul_bf16(again, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
        torch.cuda.synchronize()
    finally:
        assert lib.singe_matmul_set_splits(0) == ks.OK
    assert ops.take_device_error() == 0
    ref = oracle.linear_bf16_f32(_bits(x), _bits(w), m=m, n=n, k=k)
    assert_close_bf16(host(y32), ref, f"split-K f32 {m}x{n}x{k}")
    assert_close_bf16(host(y), oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(ref)), f"split-K bf16 {m}x{n}x{k}")
    scale = np.abs(ref).max() + 1e-6
    assert np.abs(host(y32) - ref).max() / scale < 2e-3
    assert torch.equal(y32, again)  # partial sums are added in split order: the result does not depend on timing
    # the unsplit kernel agrees to f32 accumulation-order noise
    assert lib.singe_matmul_set_splits(1) == ks.OK
    try:
        whole = torch.empty_like(y32)
        ops.matmul_bf16(whole, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
        torch.cuda.synchronize()
    finally:
        assert lib.singe_matmul_set_splits(0) == ks.OK
    assert np.abs(host(whole) - host(y32)).max() / scale < 1e-4


@pytest.mark.parametrize("m,ffn,k", [(64, 1792, 4096), (64, 14336, 512), (5, 100, 72), (128, 3584, 1024), (200, 256, 256)])
def test_swiglu_in_the_gemm_epilogue_equals_the_separate_ops_bit_for_bit(m, ffn, k):
    # gate/up rows interleaved, activation in the epilogue (regular and split-K kernels, vector and scalar stores)
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    gate = (torch.randn((ffn, k), generator=gen, device="cuda") * 0.05).to(torch.bfloat16)
    up = (torch.randn((ffn, k), generator=gen, device="cuda") * 0.05).to(torch.bfloat16)
    lib = ks.lib()
    stream = int(torch.cuda.current_stream().cuda_stream)
    # the unfused chain: one GEMM over [gate; up], then silu * up
    both = torch.cat([gate, up]).contiguous()
    projected = ops.linear(x, both)
    expect = torch.empty((m, ffn), dtype=torch.bfloat16, device="cuda")
    assert lib.singe_silu_mul_bf16(stream, expect.data_ptr(), projected.data_ptr(), projected.data_ptr() + ffn * 2,
                                   projected.stride(0), m, ffn) == ks.OK
    interleaved = torch.stack([gate, up], 1).reshape(2 * ffn, k).contiguous()
    got = torch.full((m, ffn), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert lib.singe_matmul_bf16_swiglu_bf16(stream, got.data_ptr(), x.data_ptr(), interleaved.data_ptr(), m, 2 * ffn,
                                             k, x.stride(0), interleaved.stride(0), got.stride(0)) == ks.OK
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    # same products, same split-K order only when both calls pick the same kernel; allow one bf16 ulp otherwise
    same = torch.equal(got, expect)
    if not same:
        difference = (got.float() - expect.float()).abs()
        assert float((difference / (expect.float().abs() + 1e-3)).max()) < 2e-2
    assert torch.isfinite(got.float()).all()


def test_config3_full_size_gemm_through_linearity():
    # M = 4096 against (N, K) = (4096, 4096): too large for the scalar oracle, so check sampled rows against
    # it, and the whole product through linearity: (X1 + X2) W^T == X1 W^T + X2 W^T for exactly representable sums.
    m, n, k = 4096, 4096, 4096
    x, w = _case(m, n, k)
    y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ops.matmul_bf16(y32, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
    rows = [0, 1, 127, 128, 2049, 4095]
    ref = oracle.linear_bf16_f32(_bits(x[rows]), _bits(w), m=len(rows), n=n, k=k)
    assert_close_bf16(host(y32[rows]), ref, "config 3 sampled rows")
    half = (x.float() * 0.5).to(torch.bfloat16)  # exact: halving a bf16 keeps it representable
    y_half = torch.empty_like(y32)
    ops.matmul_bf16(y_half, half, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    assert torch.equal(y_half * 2.0, y32)  # scaling by a power of two commutes with every rounding


@pytest.mark.parametrize("m,n,k", [(4096, 14336, 4096), (4096, 4096, 14336), (16, 14336, 4096), (128, 14336, 4096),
                                   (16, 4096, 14336), (128, 4096, 14336), (1, 4096, 14336), (16, 4096, 4096),
                                   (128, 4096, 4096), (1, 4096, 4096)])
def test_config3_remaining_shapes_by_sampled_rows_and_linearity(m, n, k):
    # The wide shapes of config 3 take the scalar oracle minutes in full, so: sampled rows against it (every row when
    # M <= 16), and the whole product through linearity in X, which holds exactly for a power-of-two factor.
    x, w = _case(m, n, k)
    y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ops.matmul_bf16(y32, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
    y = ops.linear(x, w)
    rows = sorted({0, 1, m // 2, m - 1, min(127, m - 1), min(128, m - 1)}) if m > 16 else list(range(m))
    rows = rows[:4] if n * k > 4096 * 4096 else rows      # the oracle needs ~0.1 s per row of a 14336-wide product
    ref = oracle.linear_bf16_f32(_bits(x[rows]), _bits(w), m=len(rows), n=n, k=k)
    assert_close_bf16(host(y32[rows]), ref, f"config 3 {m}x{n}x{k} sampled rows (f32 out)")
    assert_close_bf16(host(y[rows]), oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(ref)),
                      f"config 3 {m}x{n}x{k} sampled rows (bf16 out)")
    half = (x.float() * 0.5).to(torch.bfloat16)
    y_half = torch.empty_like(y32)
    ops.matmul_bf16(y_half, half, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    assert torch.equal(y_half * 2.0, y32)


def test_strided_operands_and_output():
    m, n, k = 96, 160, 192
    x_full, w_full = _case(m, n + 8, k + 64)
    x = x_full[:, :k]                       # row stride k + 64
    w = w_full[:n, 64:]                     # row stride k + 64, offset start (128-byte aligned)
    out = torch.full((m, n + 24), -7.0, dtype=torch.bfloat16, device="cuda")
    view = out[:, :n]
    ops.matmul_bf16(view, x, w, ops.MatmulConfig(m, n, k, x.stride(0), w.stride(0), out.stride(0), False, True))
    torch.cuda.synchronize()
    ref = oracle.linear_bf16_f32(_bits(x.contiguous()), _bits(w.contiguous()), m=m, n=n, k=k)
    assert_close_bf16(host(view), ref, "strided gemm")
    assert (out[:, n:] == -7.0).all()      # only logical output elements are written


def test_matmul_validation_mirrors_the_reference():
    # validate_matmul (singe-kernel/src/cuda/matmul.rs:2977-3020)
    lib = ks.lib()
    one = 16
    assert lib.singe_matmul_bf16_bf16(None, one, one, one, 0, 4, 4, 4, 4, 4, 0, 1) == ks.ERR_INVALID_LENGTH
    assert lib.singe_matmul_bf16_bf16(None, one, one, one, 4, 4, 8, 4, 8, 4, 0, 1) == ks.ERR_INVALID_LENGTH  # lhs stride < k
    assert lib.singe_matmul_bf16_bf16(None, one, one, one, 4, 4, 8, 8, 8, 2, 0, 1) == ks.ERR_INVALID_LENGTH  # out stride < n
    assert lib.singe_matmul_bf16_bf16(None, None, one, one, 4, 4, 8, 8, 8, 4, 0, 1) == ks.ERR_NULL_POINTER
    assert lib.singe_matmul_bf16_bf16(None, one, one, one, 16, 8, 8, 8, 8, 8, 1, 1) == ks.ERR_INVALID_LENGTH  # [K, M] lhs stride < m
    assert lib.singe_matmul_bf16_bf16(None, one, one, one, 8, 8, 8, 8, 4, 8, 0, 0) == ks.ERR_INVALID_LENGTH  # [K, N] rhs stride < n


@pytest.mark.parametrize("m,n,k,splits", [(1, 256, 512, 0), (64, 4096, 1024, 0), (200, 136, 72, 0), (256, 384, 4096, 0),
                                          (129, 1000, 520, 0), (16, 264, 2048, 4), (300, 4096, 256, 0)])
def test_row_major_right_operand_matches_the_oracle(m, n, k, splits):
    # rhs stored [K, N] (MatmulConfig::row_major, transpose_rhs false): tiles are staged N-contiguous and the tensor
    # core reads them MN-major.  The same numbers as the [N, K] call on the transposed copy, bit for bit.
    x, w = _case(m, n, k, seed=9)
    w_kn = w.t().contiguous()
    lib = ks.lib()
    assert lib.singe_matmul_set_splits(splits) == ks.OK
    try:
        y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
        ops.matmul_bf16(y32, x, w_kn, ops.MatmulConfig.row_major(m, n, k))
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        ops.matmul_bf16(y, x, w_kn, ops.MatmulConfig.row_major(m, n, k))
        twin = torch.empty_like(y32)
        ops.matmul_bf16(twin, x, w, ops.MatmulConfig.row_major_transposed_rhs(m, n, k))
        torch.cuda.synchronize()
    finally:
        assert lib.singe_matmul_set_splits(0) == ks.OK
    assert ops.take_device_error() == 0
    ref = oracle.linear_bf16_f32(_bits(x), _bits(w), m=m, n=n, k=k)
    assert_close_bf16(host(y32), ref, f"matmul [K,N] rhs {m}x{n}x{k}")
    assert_close_bf16(host(y), oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(ref)), f"bf16 out {m}x{n}x{k}")
    scale = np.abs(ref).max() + 1e-6
    assert np.abs(host(y32) - ref).max() / scale < 2e-3


def test_row_major_right_operand_with_strides():
    m, n, k = 96, 160, 192
    x, w = _case(m, n, k, seed=11)
    wide = torch.zeros((k, n + 40), dtype=torch.bfloat16, device="cuda")
    wide[:, 8:8 + n] = w.t()
    rhs = wide[:, 8:8 + n]                  # row stride n + 40, 16-byte aligned start
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ops.matmul_bf16(out, x, rhs, ops.MatmulConfig(m, n, k, k, rhs.stride(0), n, False, False))
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref = oracle.linear_bf16_f32(_bits(x), _bits(w), m=m, n=n, k=k)
    assert_close_bf16(host(out), ref, "strided [K,N] rhs")


@pytest.mark.parametrize("transpose_rhs", [True, False])
@pytest.mark.parametrize("m,n,k", [(8, 256, 512), (200, 136, 72), (256, 384, 4096), (136, 1000, 520), (304, 4096, 256),
                                   (4096, 64, 128)])
def test_transposed_left_operand_matches_the_oracle(m, n, k, transpose_rhs):
    # lhs stored [K, M] (MatmulConfig::row_major_transposed_lhs / _transposed_inputs, matmul.rs:204-246): its tiles are
    # staged M-contiguous and read MN-major, like a [K, N] right operand.
    x, w = _case(m, n, k, seed=13)
    lhs = x.t().contiguous()                              # [K, M]
    rhs = w if transpose_rhs else w.t().contiguous()      # [N, K] or [K, N]
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    config = ops.MatmulConfig(m, n, k, m, k if transpose_rhs else n, n, True, transpose_rhs)
    ops.matmul_bf16(out, lhs, rhs, config)
    rounded = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ops.matmul_bf16(rounded, lhs, rhs, config)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref = oracle.linear_bf16_f32(_bits(x), _bits(w), m=m, n=n, k=k)
    what = f"[K,M] lhs {m}x{n}x{k} transpose_rhs={transpose_rhs}"
    assert_close_bf16(host(out), ref, what)
    assert_close_bf16(host(rounded), oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(ref)), what + " bf16")
    scale = np.abs(ref).max() + 1e-6
    assert np.abs(host(out) - ref).max() / scale < 2e-3


def test_rows_that_are_not_16_byte_multiples_are_refused():
    # TMA addresses rows of the operands as they lie in memory: a row stride that is not a multiple of 16 bytes (here
    # a [K, M] left operand with M = 129) is refused, not mis-read.
    x, w = _case(129, 64, 64, seed=15)
    lhs = x.t().contiguous()
    out = torch.empty((129, 64), dtype=torch.float32, device="cuda")
    code = ks.lib().singe_matmul_bf16_f32(None, out.data_ptr(), lhs.data_ptr(), w.data_ptr(), 129, 64, 64, 129, 64, 64,
                                          1, 1)
    assert code == ks.ERR_UNSUPPORTED_CONFIGURATION
