"""The tcgen05 prefill kernel's other forms: IEEE half inputs (exact row maximum on every key tile), and the dense
[B, L, H, D] fmha_prefill_lse layout served as uniform packed sequences -- each against the CPU restatement."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops
from tests.gpu_util import assert_close_bf16, assert_close_f32, dev, dev_u32, host

pytestmark = pytest.mark.gpu

LSE_TOLERANCE = 2e-3
# f16 outputs carry 11 significant bits: tighter than the bf16 bound the shared helper applies
F16_ABS, F16_REL = 4e-3, 2e-3


def _half(rng, shape, std=1.0):
    """N(0, std) rounded to IEEE half, as f32."""
    return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float16).astype(np.float32)


def _bf16(rng, shape, std=1.0):
    return oracle.round_to_bf16(rng.standard_normal(shape, dtype=np.float32) * std).reshape(shape)


def _assert_close_f16(actual, expected, what):
    error = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    bound = F16_ABS + F16_REL * np.abs(expected)
    assert (error <= bound).all(), f"{what}: max abs err {error.max():.3e}, {(error > bound).sum()} outside the bound"


def _ragged_f16(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, causal, scale):
    total_q, total_kv = q.shape[0], k.shape[0]
    cfg = ops.RaggedKvPrefillAttentionConfig(len(lens_q), total_q, total_kv, heads, kv_heads, q.shape[2], causal, scale)
    out = torch.full((total_q, heads, q.shape[2]), float("nan"), dtype=torch.float16, device="cuda")
    lse = torch.full((total_q, heads), float("nan"), device="cuda")
    ops.ragged_kv_prefill_attention(out, lse, dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16),
                                    dev(np.asarray(lens_q, dtype=np.int32)), dev(np.asarray(lens_kv, dtype=np.int32)),
                                    dev(np.asarray(offsets, dtype=np.int32)), cfg)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    return host(out), host(lse)


def _ragged_oracle(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, causal, scale):
    return oracle.ragged_kv_prefill_attention_f32(q, k, v, lens_q, lens_kv, offsets, batch=len(lens_q),
                                                  total_query_tokens=q.shape[0], heads=heads, kv_heads=kv_heads,
                                                  head_dim=q.shape[2], causal=causal, scale=scale)


@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lens", [[5], [129, 1], [300, 127, 256, 1], [1000, 40]])
def test_ragged_prefill_f16_matches_the_oracle(causal, lens, head_dim):
    heads, kv_heads = 4, 2
    rng = np.random.default_rng(300 + sum(lens))
    total = sum(lens)
    q, k, v = (_half(rng, (total, heads, head_dim)), _half(rng, (total, kv_heads, head_dim)),
               _half(rng, (total, kv_heads, head_dim)))
    offsets = np.concatenate([[0], np.cumsum(lens)[:-1]])
    scale = 1.0 / np.sqrt(head_dim)
    out, lse = _ragged_f16(q, k, v, lens, lens, offsets, heads, kv_heads, causal, scale)
    ref_out, ref_lse = _ragged_oracle(q, k, v, lens, lens, offsets, heads, kv_heads, causal, scale)
    _assert_close_f16(out, ref_out, f"f16 prefill out lens={lens} causal={causal}")
    assert_close_f32(lse, ref_lse, f"f16 prefill lse lens={lens} causal={causal}", LSE_TOLERANCE)


def test_f16_prefill_keeps_probabilities_in_the_half_range_when_scores_climb():
    # Keys grow in norm along the sequence and one block is far larger: a softmax relative to the first tile's
    # maximum would need probabilities beyond 65504.  Every tile takes its own exact maximum instead.
    rng = np.random.default_rng(41)
    heads, kv_heads = 4, 2
    lens = [600, 300]
    total = sum(lens)
    q = _half(rng, (total, heads, 128))
    k = rng.standard_normal((total, kv_heads, 128), dtype=np.float32)
    k[300:600] *= 12.0
    k = k.astype(np.float16).astype(np.float32)
    v = _half(rng, (total, kv_heads, 128))
    for causal in (True, False):
        out, lse = _ragged_f16(q, k, v, lens, lens, [0, 600], heads, kv_heads, causal, 1.0)
        ref_out, ref_lse = _ragged_oracle(q, k, v, lens, lens, [0, 600], heads, kv_heads, causal, 1.0)
        assert np.isfinite(out).all() and np.isfinite(lse).all()
        _assert_close_f16(out, ref_out, f"f16 out across a score jump, causal={causal}")
        assert np.allclose(lse, ref_lse, rtol=1e-5, atol=5e-3)


def test_f16_prefill_with_different_query_and_key_lengths_and_an_empty_sequence():
    rng = np.random.default_rng(43)
    heads, kv_heads = 4, 4
    lens_q, lens_kv, offsets = [200, 60, 30], [100, 260, 0], [0, 270, 540]
    total = 580
    q, k, v = _half(rng, (total, heads, 128)), _half(rng, (total, kv_heads, 128)), _half(rng, (total, kv_heads, 128))
    scale = 0.11
    out, lse = _ragged_f16(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, True, scale)
    ref_out, ref_lse = _ragged_oracle(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, True, scale)
    rows = np.concatenate([np.arange(o, o + n) for o, n in zip(offsets, lens_q)])
    _assert_close_f16(out[rows], ref_out[rows], "f16 out, lens differ")
    assert_close_f32(lse[rows], ref_lse[rows], "f16 lse, lens differ", LSE_TOLERANCE)
    assert (out[540:570] == 0).all() and (lse[540:570] == np.float32(-1.0e20)).all()  # no keys: zeros, empty LSE
    gap = np.setdiff1d(np.arange(total), rows)
    assert np.isnan(out[gap]).all() and np.isnan(lse[gap]).all()                     # rows nobody owns stay untouched


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lens", [[300, 127, 256, 1], [1000, 40]])
def test_ragged_prefill_bf16_head_dim_64_on_the_tensor_core(causal, lens):
    heads, kv_heads = 8, 2
    rng = np.random.default_rng(350 + sum(lens))
    total = sum(lens)
    q, k, v = _bf16(rng, (total, heads, 64)), _bf16(rng, (total, kv_heads, 64)), _bf16(rng, (total, kv_heads, 64))
    offsets = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    cfg = ops.RaggedKvPrefillAttentionConfig(len(lens), total, total, heads, kv_heads, 64, causal, 0.125)
    out = torch.full((total, heads, 64), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((total, heads), float("nan"), device="cuda")
    ops.ragged_kv_prefill_attention(out, lse, dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16),
                                    dev(np.asarray(lens, dtype=np.int32)), dev(np.asarray(lens, dtype=np.int32)),
                                    dev(offsets), cfg)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref_out, ref_lse = _ragged_oracle(q, k, v, lens, lens, offsets, heads, kv_heads, causal, 0.125)
    assert_close_bf16(host(out), ref_out, f"bf16 head_dim 64 out lens={lens} causal={causal}")
    assert_close_f32(host(lse), ref_lse, f"bf16 head_dim 64 lse lens={lens} causal={causal}", LSE_TOLERANCE)


@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
def test_paged_prefill_f16_through_the_block_table(causal, head_dim):
    rng = np.random.default_rng(47)
    heads, kv_heads, block = 8, 2, 16
    lens_q = np.array([300, 1, 129, 40, 257], dtype=np.int32)
    lens_kv = np.array([300, 517, 100, 0, 257], dtype=np.int32)
    offsets = np.concatenate([[0], np.cumsum(lens_q)[:-1]]).astype(np.int32)
    total = int(lens_q.sum())
    stride = 40
    pages_per = (lens_kv + block - 1) // block
    pool = int(pages_per.sum()) + 5
    perm = rng.permutation(pool).astype(np.uint32)
    table = np.zeros((len(lens_q), stride), dtype=np.uint32)
    at = 0
    for b, n in enumerate(pages_per):
        table[b, :n] = perm[at: at + n]
        at += int(n)
    q = _half(rng, (total, heads, head_dim))
    kc = _half(rng, (pool, block, kv_heads, head_dim))
    vc = _half(rng, (pool, block, kv_heads, head_dim))
    scale = 1.0 / np.sqrt(head_dim)
    cfg = ops.PagedKvPrefillAttentionConfig(len(lens_q), total, heads, kv_heads, head_dim, block, pool, stride, causal,
                                            scale)
    out = torch.full((total, heads, head_dim), 7.0, dtype=torch.float16, device="cuda")
    lse = torch.full((total, heads), 7.0, device="cuda")
    ops.paged_kv_prefill_attention(out, lse, dev(q, torch.float16), dev(kc, torch.float16), dev(vc, torch.float16),
                                   dev(lens_q), dev(lens_kv), dev(offsets), dev_u32(table), cfg)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref_out, ref_lse = oracle.paged_kv_prefill_attention_f32(
        q, kc, vc, lens_q, lens_kv, offsets, table, batch=len(lens_q), total_query_tokens=total, heads=heads,
        kv_heads=kv_heads, head_dim=head_dim, block_size=block, block_table_batch_stride=stride, causal=causal,
        scale=scale)
    _assert_close_f16(host(out), ref_out, f"paged prefill f16 out causal={causal}")
    assert_close_f32(host(lse), ref_lse, f"paged prefill f16 lse causal={causal}", LSE_TOLERANCE)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("batch,query_len,key_len,heads,kv_heads,head_dim",
                         [(2, 300, 420, 4, 2, 128), (3, 257, 257, 2, 2, 128), (1, 520, 130, 4, 1, 128),
                          (2, 300, 200, 4, 2, 64), (2, 40, 56, 4, 2, 32)])
def test_dense_prefill_with_lse_on_16_bit_floats(dtype, causal, batch, query_len, key_len, heads, kv_heads, head_dim):
    # fmha_prefill_lse_{bf16,f16}: [B, L, H, D] over [B, S, G, D], lse [B, H, L]; causal hides key > query index.
    # head_dim 128 and 64 run the tensor-core kernel's dense form, other widths the general kernel.
    rng = np.random.default_rng(500 + query_len + key_len)
    make = _bf16 if dtype == torch.bfloat16 else _half
    q = make(rng, (batch, query_len, heads, head_dim))
    k = make(rng, (batch, key_len, kv_heads, head_dim))
    v = make(rng, (batch, key_len, kv_heads, head_dim))
    scale = 1.0 / np.sqrt(head_dim)
    out = torch.full((batch, query_len, heads, head_dim), float("nan"), dtype=dtype, device="cuda")
    lse = torch.full((batch, heads, query_len), float("nan"), device="cuda")
    ops.fmha_prefill_lse(out, lse, dev(q, dtype), dev(k, dtype), dev(v, dtype), batch=batch, query_len=query_len,
                         key_len=key_len, heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale,
                         causal=causal)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref_out, ref_lse = oracle.fmha_prefill_lse_f32(q, k, v, batch=batch, query_len=query_len, key_len=key_len,
                                                   heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale,
                                                   causal=causal)
    what = f"dense prefill {dtype} {batch}x{query_len}x{key_len} d{head_dim} causal={causal}"
    if dtype == torch.bfloat16:
        assert_close_bf16(host(out), ref_out, what)
    else:
        _assert_close_f16(host(out), ref_out, what)
    assert_close_f32(host(lse), ref_lse.reshape(batch, heads, query_len), what + " lse", LSE_TOLERANCE)
