"""Packed variable-length prefill (tcgen05 kernel for bf16 / head_dim 128) against the CPU restatement of
ragged_kv_prefill_attention_f32, and the fused slot-mapped cache write."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops, workloads
from tests.gpu_util import assert_close_bf16, assert_close_f32, dev, host

pytestmark = pytest.mark.gpu

LSE_TOLERANCE = 2e-3  # natural-log LSE from exp2-domain f32 sums


def _run(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, causal, scale, cache_write=None):
    total_q, total_kv = q.shape[0], k.shape[0]
    cfg = ops.RaggedKvPrefillAttentionConfig(len(lens_q), total_q, total_kv, heads, kv_heads, q.shape[2], causal,
                                             scale)
    out = torch.full((total_q, heads, q.shape[2]), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((total_q, heads), float("nan"), device="cuda")
    ops.ragged_kv_prefill_attention(out, lse, dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16),
                                    dev(np.asarray(lens_q, dtype=np.int32)), dev(np.asarray(lens_kv, dtype=np.int32)),
                                    dev(np.asarray(offsets, dtype=np.int32)), cfg, cache_write=cache_write)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    return host(out), host(lse)


def _oracle(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, causal, scale):
    return oracle.ragged_kv_prefill_attention_f32(q, k, v, lens_q, lens_kv, offsets, batch=len(lens_q),
                                                  total_query_tokens=q.shape[0], heads=heads, kv_heads=kv_heads,
                                                  head_dim=q.shape[2], causal=causal, scale=scale)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lens", [[5], [128], [129, 1], [300, 127, 256, 1], [1000, 40]])
@pytest.mark.parametrize("heads,kv_heads", [(4, 2), (2, 2), (8, 1)])
def test_ragged_prefill_bf16_matches_the_oracle(causal, lens, heads, kv_heads):
    rng = np.random.default_rng(100 + sum(lens) + heads)
    total = sum(lens)
    q = workloads.normal_bf16(rng, (total, heads, 128))
    k = workloads.normal_bf16(rng, (total, kv_heads, 128))
    v = workloads.normal_bf16(rng, (total, kv_heads, 128))
    offsets = np.concatenate([[0], np.cumsum(lens)[:-1]])
    scale = 1.0 / np.sqrt(128.0)
    out, lse = _run(q, k, v, lens, lens, offsets, heads, kv_heads, causal, scale)
    ref_out, ref_lse = _oracle(q, k, v, lens, lens, offsets, heads, kv_heads, causal, scale)
    assert_close_bf16(out, ref_out, f"prefill out lens={lens} causal={causal}")
    assert_close_f32(lse, ref_lse, f"prefill lse lens={lens} causal={causal}", LSE_TOLERANCE)


def test_query_and_key_lengths_may_differ_and_gaps_stay_untouched():
    # Sequence 0: 200 queries over 100 keys; sequence 1: 60 queries over 260 keys; 10 unused rows between them.
    # Causal hides key_index > query_index with sequence-local indices and no offset (cpu/attention.rs:1377).
    rng = np.random.default_rng(7)
    heads, kv_heads = 4, 4
    lens_q, lens_kv, offsets = [200, 60], [100, 260], [0, 270]
    total = 270 + 260
    q = workloads.normal_bf16(rng, (total, heads, 128))
    k = workloads.normal_bf16(rng, (total, kv_heads, 128))
    v = workloads.normal_bf16(rng, (total, kv_heads, 128))
    for causal in (True, False):
        out, lse = _run(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, causal, 0.09)
        ref_out, ref_lse = _oracle(q, k, v, lens_q, lens_kv, offsets, heads, kv_heads, causal, 0.09)
        owned = np.zeros(total, dtype=bool)
        owned[0:200] = True
        owned[270:330] = True
        assert_close_bf16(out[owned], ref_out[owned], f"out causal={causal}")
        assert_close_f32(lse[owned], ref_lse[owned], f"lse causal={causal}", LSE_TOLERANCE)
        assert np.isnan(out[~owned]).all() and np.isnan(lse[~owned]).all()  # only logical elements are written


def test_a_sequence_without_keys_gets_zeros_and_the_empty_lse():
    rng = np.random.default_rng(8)
    lens_q, lens_kv, offsets = [130, 3], [0, 3], [0, 130]
    q = workloads.normal_bf16(rng, (133, 2, 128))
    k = workloads.normal_bf16(rng, (133, 2, 128))
    v = workloads.normal_bf16(rng, (133, 2, 128))
    out, lse = _run(q, k, v, lens_q, lens_kv, offsets, 2, 2, True, 0.1)
    ref_out, ref_lse = _oracle(q, k, v, lens_q, lens_kv, offsets, 2, 2, True, 0.1)
    assert not out[:130].any() and (lse[:130] == np.float32(-1.0e20)).all()
    assert_close_bf16(out, ref_out, "out")
    assert_close_f32(lse[130:], ref_lse[130:], "lse", LSE_TOLERANCE)


def test_large_scores_exercise_the_lazy_rescale():
    # Keys grow in norm along the sequence, so the running max keeps rising by far more than the rescale threshold.
    rng = np.random.default_rng(9)
    n, heads = 700, 2
    q = workloads.normal_bf16(rng, (n, heads, 128))
    ramp = np.linspace(0.2, 6.0, n, dtype=np.float32)[:, None, None]
    k = oracle.round_to_bf16(rng.standard_normal((n, heads, 128), dtype=np.float32) * ramp).reshape(n, heads, 128)
    v = workloads.normal_bf16(rng, (n, heads, 128))
    out, lse = _run(q, k, v, [n], [n], [0], heads, heads, True, 0.25)
    ref_out, ref_lse = _oracle(q, k, v, [n], [n], [0], heads, heads, True, 0.25)
    assert_close_bf16(out, ref_out, "out under large scores")
    assert_close_f32(lse, ref_lse, "lse under large scores", 5e-3)


def test_a_score_jump_beyond_the_single_pass_range_is_redone_exactly():
    # After the first key tile the kernel keeps no row maximum; a row whose scores jump by more than 2^64 between key
    # tiles leaves that scheme's range and its CTA is recomputed with exact maxima.  Keys from index 300 on are 12x
    # larger, so with scale 1 the later tiles' scores exceed the earlier ones by hundreds of log2 units.  The second
    # sequence stays in range and shares the launch.
    rng = np.random.default_rng(11)
    heads, kv_heads = 4, 2
    lens = [600, 300]
    total = sum(lens)
    q = workloads.normal_bf16(rng, (total, heads, 128))
    k = rng.standard_normal((total, kv_heads, 128), dtype=np.float32)
    k[300:600] *= 12.0
    k = oracle.round_to_bf16(k).reshape(total, kv_heads, 128)
    v = workloads.normal_bf16(rng, (total, kv_heads, 128))
    for causal in (True, False):
        out, lse = _run(q, k, v, lens, lens, [0, 600], heads, kv_heads, causal, 1.0)
        ref_out, ref_lse = _oracle(q, k, v, lens, lens, [0, 600], heads, kv_heads, causal, 1.0)
        assert np.isfinite(out).all() and np.isfinite(lse).all()
        assert_close_bf16(out, ref_out, f"out across a score jump, causal={causal}")
        assert np.allclose(lse, ref_lse, rtol=1e-5, atol=5e-3), "lse across a score jump"


def test_config4_prefill_with_the_cache_write_in_the_same_call():
    # lengths {8192, 4096, 2048, 1024}, 32 Q / 8 KV heads, head_dim 128, seed 3, causal; K/V also stored into 16-token
    # pages of a permuted pool.  The scalar oracle covers the whole 1024-token sequence; rows of the longer
    # sequences are sampled (tile edges, first and last rows) against a float64 evaluation of the same formula.
    case = workloads.prefill_case()
    rng = np.random.default_rng(3)
    total = case.total_tokens
    q = workloads.normal_bf16(rng, (total, case.heads, case.head_dim))
    k = workloads.normal_bf16(rng, (total, case.kv_heads, case.head_dim))
    v = workloads.normal_bf16(rng, (total, case.kv_heads, case.head_dim))
    shape = (case.pages, case.page_size, case.kv_heads, case.head_dim)
    key_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    value_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = _run(q, k, v, case.lens, case.lens, case.offsets, case.heads, case.kv_heads, True, case.scale,
                    cache_write=(key_cache, value_cache, dev(case.write_pages), dev(case.write_slots), status))
    assert int(status.item()) == 0
    # cache contents: bit-exact against the oracle's slot-mapped write
    expect_k = np.zeros(shape, dtype=np.float32)
    expect_v = np.zeros(shape, dtype=np.float32)
    assert oracle.kv_cache_write(expect_k, k, case.write_pages, case.write_slots) == oracle.OK
    assert oracle.kv_cache_write(expect_v, v, case.write_pages, case.write_slots) == oracle.OK
    assert np.array_equal(host(key_cache), expect_k) and np.array_equal(host(value_cache), expect_v)
    # the 1024-token sequence, every head, through the oracle
    first, n = int(case.offsets[3]), int(case.lens[3])
    ref_out, ref_lse = _oracle(q[first:first + n], k[first:first + n], v[first:first + n], [n], [n], [0], case.heads,
                               case.kv_heads, True, case.scale)
    assert_close_bf16(out[first:first + n], ref_out, "config 4, sequence of 1024")
    assert_close_f32(lse[first:first + n], ref_lse, "config 4 lse, sequence of 1024", LSE_TOLERANCE)
    # sampled rows of the longer sequences
    group = case.heads // case.kv_heads
    for b in range(3):
        base, length = int(case.offsets[b]), int(case.lens[b])
        for i in sorted({0, 1, 127, 128, 129, length // 2, length - 129, length - 128, length - 1}):
            for h in (0, 13, 31):
                keys = k[base:base + i + 1, h // group].astype(np.float64)
                vals = v[base:base + i + 1, h // group].astype(np.float64)
                s = keys @ q[base + i, h].astype(np.float64) * case.scale
                w = np.exp(s - s.max())
                expect = (w / w.sum()) @ vals
                error = np.abs(out[base + i, h] - expect)
                assert (error <= 2e-2 + 1e-2 * np.abs(expect)).all(), f"seq {b} row {i} head {h}: {error.max():.3e}"
                assert abs(lse[base + i, h] - (s.max() + np.log(w.sum()))) < LSE_TOLERANCE
    assert not np.isnan(out).any() and not np.isnan(lse).any()
