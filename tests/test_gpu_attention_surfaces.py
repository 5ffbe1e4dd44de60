"""Dense, packed-prefill and Tensor-surface paged attention on the GPU against the CPU restatements."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops, workloads
from tests.gpu_util import assert_close_bf16, assert_close_f32, dev, dev_u32, host

pytestmark = pytest.mark.gpu


def test_config1_causal_sdpa_f32_matches_the_reference_cpu_kernel():
    # Config 1: batch 1, 8 heads, seq 512, head_dim 64, N(0,1) seed 0, scale 1/8, causal -> [1,8,512,64] f32.
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((1, 8, 512, 64), dtype=np.float32) for _ in range(3))
    got = ops.scaled_dot_product_attention(dev(q), dev(k), dev(v), scale=1.0 / 8.0, causal=True)
    torch.cuda.synchronize()
    ref = oracle.scaled_dot_product_attention_f32(q, k, v, scale=1.0 / 8.0, causal=True)
    assert got.shape == (1, 8, 512, 64)
    assert_close_f32(host(got), ref, "config 1 SDPA")


def test_sdpa_gqa_window_and_non_causal():
    rng = np.random.default_rng(5)
    q = rng.standard_normal((2, 4, 33, 16), dtype=np.float32)
    k = rng.standard_normal((2, 2, 40, 16), dtype=np.float32)
    v = rng.standard_normal((2, 2, 40, 16), dtype=np.float32)
    rep = lambda x: np.repeat(x, 2, axis=1)  # repeat_kv (singe/src/backend/cpu/normalization/attention.rs:20-130)
    for causal, window in [(False, 0), (True, 0), (True, 5)]:
        got = ops.scaled_dot_product_attention(dev(q), dev(k), dev(v), scale=0.25, causal=causal, window=window)
        ref = oracle.scaled_dot_product_attention_f32(q, rep(k), rep(v), scale=0.25, causal=causal, window=window)
        assert_close_f32(host(got), ref, f"sdpa causal={causal} window={window}")


def test_fmha_prefill_lse_f32():
    rng = np.random.default_rng(6)
    b, l, s, h, g, d = 2, 19, 19, 4, 2, 32
    q = rng.standard_normal((b, l, h, d), dtype=np.float32)
    k = rng.standard_normal((b, s, g, d), dtype=np.float32)
    v = rng.standard_normal((b, s, g, d), dtype=np.float32)
    out = torch.empty((b, l, h, d), device="cuda")
    lse = torch.empty((b, h, l), device="cuda")
    ops.fmha_prefill_lse(out, lse, dev(q), dev(k), dev(v), batch=b, query_len=l, key_len=s, heads=h, kv_heads=g,
                         head_dim=d, scale=0.2, causal=True)
    ref_out, ref_lse = oracle.fmha_prefill_lse_f32(q, k, v, batch=b, query_len=l, key_len=s, heads=h, kv_heads=g,
                                                   head_dim=d, scale=0.2, causal=True)
    assert_close_f32(host(out), ref_out, "fmha_prefill out")
    assert_close_f32(host(lse), ref_lse, "fmha_prefill lse")


def _ragged_case(rng, lens, heads, kv_heads, head_dim, bf16):
    total = int(sum(lens))
    make = (lambda shape: workloads.normal_bf16(rng, shape)) if bf16 else (
        lambda shape: rng.standard_normal(shape, dtype=np.float32))
    q = make((total, heads, head_dim))
    k = make((total, kv_heads, head_dim))
    v = make((total, kv_heads, head_dim))
    offsets = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    return q, k, v, np.asarray(lens, dtype=np.int32), offsets


@pytest.mark.parametrize("causal", [True, False])
def test_ragged_prefill_f32_general_kernel(causal):
    rng = np.random.default_rng(7)
    lens = [5, 1, 40]
    heads, kv_heads, head_dim = 4, 2, 24
    q, k, v, lens_np, offsets = _ragged_case(rng, lens, heads, kv_heads, head_dim, bf16=False)
    total = int(lens_np.sum())
    cfg = ops.RaggedKvPrefillAttentionConfig(3, total, total, heads, kv_heads, head_dim, causal, 0.3)
    out = torch.zeros((total, heads, head_dim), device="cuda")
    lse = torch.zeros((total, heads), device="cuda")
    ops.ragged_kv_prefill_attention(out, lse, dev(q), dev(k), dev(v), dev(lens_np), dev(lens_np), dev(offsets), cfg)
    ref_out, ref_lse = oracle.ragged_kv_prefill_attention_f32(q, k, v, lens_np, lens_np, offsets, batch=3,
                                                              total_query_tokens=total, heads=heads,
                                                              kv_heads=kv_heads, head_dim=head_dim, causal=causal,
                                                              scale=0.3)
    assert_close_f32(host(out), ref_out, "ragged prefill out")
    assert_close_f32(host(lse), ref_lse, "ragged prefill lse")


def test_paged_prefill_f32_and_empty_rows():
    # len_kv == 0 for one sequence: rows that see no key get out = 0 and lse = -1e20 (cpu/attention.rs:1304)
    rng = np.random.default_rng(8)
    heads, kv_heads, head_dim, block = 4, 2, 16, 4
    lens_q = np.array([6, 2, 3], dtype=np.int32)
    lens_kv = np.array([6, 0, 9], dtype=np.int32)
    offsets = np.array([0, 6, 8], dtype=np.int32)
    total = 11
    pool, stride = 8, 3
    perm = rng.permutation(pool).astype(np.uint32)
    table = np.zeros((3, stride), dtype=np.uint32)
    table[0, :2] = perm[:2]
    table[2, :3] = perm[2:5]
    q = rng.standard_normal((total, heads, head_dim), dtype=np.float32)
    kc = rng.standard_normal((pool, block, kv_heads, head_dim), dtype=np.float32)
    vc = rng.standard_normal((pool, block, kv_heads, head_dim), dtype=np.float32)
    for causal in (True, False):
        cfg = ops.PagedKvPrefillAttentionConfig(3, total, heads, kv_heads, head_dim, block, pool, stride, causal, 0.25)
        out = torch.full((total, heads, head_dim), 7.0, device="cuda")
        lse = torch.full((total, heads), 7.0, device="cuda")
        ops.paged_kv_prefill_attention(out, lse, dev(q), dev(kc), dev(vc), dev(lens_q), dev(lens_kv), dev(offsets),
                                       dev_u32(table), cfg)
        ref_out, ref_lse = oracle.paged_kv_prefill_attention_f32(
            q, kc, vc, lens_q, lens_kv, offsets, table, batch=3, total_query_tokens=total, heads=heads,
            kv_heads=kv_heads, head_dim=head_dim, block_size=block, block_table_batch_stride=stride, causal=causal,
            scale=0.25)
        assert_close_f32(host(out), ref_out, f"paged prefill out causal={causal}")
        assert_close_f32(host(lse), ref_lse, f"paged prefill lse causal={causal}")


# ---- Tensor-surface paged attention: singe/tests/nn/paged_attention.rs ----
TOKENS, HEADS, DIM, SLOTS, PAGES = 2, 2, 16, 4, 2
VALID = dict(query_offsets=[0, 2], page_offsets=[0, 1], pages=[0], last_page_lengths=[2])
INVALID = [
    dict(VALID, query_offsets=[0, 3]), dict(VALID, query_offsets=[-1, 2]), dict(VALID, query_offsets=[2, 0]),
    dict(VALID, page_offsets=[0, 2]), dict(VALID, page_offsets=[-1, 1]), dict(VALID, pages=[PAGES]),
    dict(VALID, pages=[-1]), dict(VALID, last_page_lengths=[SLOTS + 1]), dict(VALID, last_page_lengths=[-1]),
]


def _attend(paging, dtype, index_dtype=np.int64):
    q = torch.zeros((TOKENS, HEADS, DIM), dtype=dtype, device="cuda")
    cache = torch.zeros((PAGES, SLOTS, HEADS, DIM), dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    idx = {name: dev(np.asarray(values, dtype=index_dtype)) for name, values in paging.items()}
    out, lse = ops.paged_attention(q, cache, cache, idx["query_offsets"], idx["page_offsets"], idx["pages"],
                                   idx["last_page_lengths"], causal=True, status=status)
    torch.cuda.synchronize()
    return int(status.item()), out, lse


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("index_dtype", [np.int64, np.int32])
def test_paging_values_outside_their_buffers_set_the_status_word_and_never_fault(dtype, index_dtype):
    # singe/tests/nn/paged_attention.rs:145-184: nine invalid tuples -> IndexOutOfBounds, two valid edge cases.
    status, out, lse = _attend(VALID, dtype, index_dtype)
    assert status == 0
    assert np.allclose(host(lse)[:, 0], [0.0, 1.0])  # zero scores: log2 of 1 and 2 visible keys
    for paging in INVALID:
        assert _attend(paging, dtype, index_dtype)[0] == 1, paging
    assert _attend(dict(VALID, last_page_lengths=[SLOTS]), dtype, index_dtype)[0] == 0
    assert _attend(dict(query_offsets=[0, 0], page_offsets=[0, 0], pages=[PAGES + 7], last_page_lengths=[-1]),
                   dtype, index_dtype)[0] == 0


@pytest.mark.parametrize("dtype,bf16", [(torch.float32, False), (torch.bfloat16, True)])
def test_tensor_paged_attention_mixes_prefill_and_decode_rows(dtype, bf16):
    # Three sequences: a prompt of 7 tokens, a single decode token over 21 keys, and 3 new tokens over 12 keys.
    rng = np.random.default_rng(9)
    heads, kv_heads, head_dim, page = 4, 2, 32, 4
    keys = [7, 21, 12]
    queries = [7, 1, 3]
    pages_per = [(n + page - 1) // page for n in keys]
    pool = sum(pages_per) + 2
    perm = rng.permutation(pool)
    pages = perm[: sum(pages_per)]
    page_offsets = np.concatenate([[0], np.cumsum(pages_per)])
    query_offsets = np.concatenate([[0], np.cumsum(queries)])
    last = [(n - 1) % page + 1 for n in keys]
    total = sum(queries)
    make = (lambda shape: workloads.normal_bf16(rng, shape)) if bf16 else (
        lambda shape: rng.standard_normal(shape, dtype=np.float32))
    q = make((total, heads, head_dim))
    kc = make((pool, page, kv_heads, head_dim))
    vc = make((pool, page, kv_heads, head_dim))
    for causal, window in [(True, 0), (True, 6), (False, 0)]:
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out, lse = ops.paged_attention(dev(q, dtype), dev(kc, dtype), dev(vc, dtype), dev(query_offsets),
                                       dev(page_offsets), dev(pages.astype(np.int64)),
                                       dev(np.asarray(last, dtype=np.int64)), scale=0.2, causal=causal,
                                       window=window, status=status)
        code, ref_out, ref_lse = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last,
                                                         scale=0.2, causal=causal, window=window)
        assert code == oracle.OK and int(status.item()) == 0
        if bf16:
            assert_close_bf16(host(out), ref_out, f"tensor paged bf16 causal={causal} window={window}")
        else:
            assert_close_f32(host(out), ref_out, f"tensor paged out causal={causal} window={window}")
        assert_close_f32(host(lse), ref_lse, "tensor paged lse (base 2)", 2e-4)


def _decode_batch(rng, lens, heads, kv_heads, page=16, head_dim=128, spare=3):
    pages_per = [(n + page - 1) // page for n in lens]
    pool = sum(pages_per) + spare
    pages = rng.permutation(pool)[: sum(pages_per)].astype(np.int64)
    page_offsets = np.concatenate([[0], np.cumsum(pages_per)]).astype(np.int64)
    last = np.asarray([(n - 1) % page + 1 if n > 0 else 0 for n in lens], dtype=np.int64)
    q = workloads.normal_bf16(rng, (len(lens), heads, head_dim))
    kc = workloads.normal_bf16(rng, (pool, page, kv_heads, head_dim))
    vc = workloads.normal_bf16(rng, (pool, page, kv_heads, head_dim))
    return q, kc, vc, pages, page_offsets, last


@pytest.mark.parametrize("index_dtype", [np.int64, np.int32])
@pytest.mark.parametrize("lens", [[1, 700, 16, 0, 2049, 513], [4096, 128], [33] * 40])
def test_a_plain_decode_batch_through_the_tensor_surface_takes_the_tiled_kernel_and_matches(lens, index_dtype):
    # One query token per sequence, bf16, head_dim 128, 16-token pages: the planning kernel hands the call to the
    # tiled flash-decode kernel (split-K for the long sequences, zeros and -inf for the empty one); out and the base-2
    # LSE must match the CPU restatement of attend_paged like any other call.
    rng = np.random.default_rng(31 + len(lens))
    heads, kv_heads = 8, 2
    q, kc, vc, pages, page_offsets, last = _decode_batch(rng, lens, heads, kv_heads)
    query_offsets = np.arange(len(lens) + 1, dtype=np.int64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cast = lambda a: dev(np.asarray(a, dtype=index_dtype))
    scale = 1.0 / np.sqrt(128.0)
    out, lse = ops.paged_attention(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16),
                                   cast(query_offsets), cast(page_offsets), cast(pages), cast(last), scale=scale,
                                   causal=True, status=status)
    torch.cuda.synchronize()
    code, ref_out, ref_lse = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last, scale=scale,
                                                     causal=True)
    assert code == oracle.OK and int(status.item()) == 0 and ops.take_device_error() == 0
    assert_close_bf16(host(out), ref_out, f"tensor-surface decode out lens={lens[:4]}")
    got_lse, finite = host(lse), np.isfinite(ref_lse)
    assert (np.isneginf(got_lse) == np.isneginf(ref_lse)).all()
    assert np.abs(got_lse[finite] - ref_lse[finite]).max() < 5e-3


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("window", [1, 5, 16, 17, 100, 1000, 5000])
def test_a_plain_decode_batch_with_a_sliding_window_stays_on_the_tiled_kernel(window, causal):
    # The planning kernel drops the whole pages in front of the window (key-tile skipping) and tells the tiled kernel
    # how many keys at the front of the first remaining page are still hidden.  The query at position keys - 1 sees
    # keys >= keys - window whether the call is causal or not.  Windows of one key, inside one page, exactly a page,
    # across pages and splits, and wider than every sequence.
    rng = np.random.default_rng(70 + window)
    heads, kv_heads = 8, 2
    lens = [1, 700, 16, 0, 2049, 513, 17, 31]
    q, kc, vc, pages, page_offsets, last = _decode_batch(rng, lens, heads, kv_heads)
    query_offsets = np.arange(len(lens) + 1, dtype=np.int64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = 1.0 / np.sqrt(128.0)
    out, lse = ops.paged_attention(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16),
                                   dev(query_offsets), dev(page_offsets), dev(pages), dev(last), scale=scale,
                                   causal=causal, window=window, status=status)
    torch.cuda.synchronize()
    code, ref_out, ref_lse = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last, scale=scale,
                                                     causal=causal, window=window)
    assert code == oracle.OK and int(status.item()) == 0 and ops.take_device_error() == 0
    assert_close_bf16(host(out), ref_out, f"windowed tensor-surface decode, window={window} causal={causal}")
    got_lse, finite = host(lse), np.isfinite(ref_lse)
    assert (np.isneginf(got_lse) == np.isneginf(ref_lse)).all()
    assert np.abs(got_lse[finite] - ref_lse[finite]).max() < 5e-3
    if window < 500:
        full = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last, scale=scale, causal=causal)[1]
        assert np.abs(full - ref_out).max() > 1e-2   # the window changes the answer


def test_a_batch_that_only_looks_like_decode_is_left_to_the_general_kernel():
    # tokens == sequences, but sequence 0 owns two query tokens and sequence 1 none: the planning kernel must not hand
    # this to the tiled kernel.  Then a bad page id in an otherwise plain decode batch: status 1, no fault.
    rng = np.random.default_rng(41)
    heads, kv_heads = 8, 2
    lens = [40, 0, 300]
    q, kc, vc, pages, page_offsets, last = _decode_batch(rng, lens, heads, kv_heads)
    query_offsets = np.asarray([0, 2, 2, 3], dtype=np.int64)
    scale = 0.1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = ops.paged_attention(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16),
                                   dev(query_offsets), dev(page_offsets), dev(pages), dev(last), scale=scale,
                                   causal=True, status=status)
    code, ref_out, ref_lse = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last, scale=scale,
                                                     causal=True)
    assert code == oracle.OK and int(status.item()) == 0
    assert_close_bf16(host(out), ref_out, "two queries in one sequence")
    finite = np.isfinite(ref_lse)
    assert np.abs(host(lse)[finite] - ref_lse[finite]).max() < 5e-3
    bad = pages.copy()
    bad[5] = kc.shape[0]  # one past the cache
    status.zero_()
    ops.paged_attention(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16),
                        dev(np.arange(4, dtype=np.int64)), dev(page_offsets), dev(bad), dev(last), scale=scale,
                        causal=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 1


@pytest.mark.parametrize("causal", [True, False])
def test_paged_prefill_bf16_gathers_its_key_tiles_through_the_block_table(causal):
    # bf16, head_dim 128, 16-token pages: the tensor-core prefill kernel reads K and V page by page from a permuted
    # pool.  Sequences with more keys than queries, fewer keys than queries, no keys at all, and a ragged last page.
    rng = np.random.default_rng(51)
    heads, kv_heads, head_dim, block = 8, 2, 128, 16
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
    q = workloads.normal_bf16(rng, (total, heads, head_dim))
    kc = workloads.normal_bf16(rng, (pool, block, kv_heads, head_dim))
    vc = workloads.normal_bf16(rng, (pool, block, kv_heads, head_dim))
    scale = 1.0 / np.sqrt(128.0)
    cfg = ops.PagedKvPrefillAttentionConfig(len(lens_q), total, heads, kv_heads, head_dim, block, pool, stride, causal,
                                            scale)
    out = torch.full((total, heads, head_dim), 7.0, dtype=torch.bfloat16, device="cuda")
    lse = torch.full((total, heads), 7.0, device="cuda")
    ops.paged_kv_prefill_attention(out, lse, dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16),
                                   dev(lens_q), dev(lens_kv), dev(offsets), dev_u32(table), cfg)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref_out, ref_lse = oracle.paged_kv_prefill_attention_f32(
        q, kc, vc, lens_q, lens_kv, offsets, table, batch=len(lens_q), total_query_tokens=total, heads=heads,
        kv_heads=kv_heads, head_dim=head_dim, block_size=block, block_table_batch_stride=stride, causal=causal,
        scale=scale)
    assert_close_bf16(host(out), ref_out, f"paged prefill bf16 out causal={causal}")
    assert_close_f32(host(lse), ref_lse, f"paged prefill bf16 lse causal={causal}", 2e-3)


def test_attend_with_a_score_cap_and_per_head_sinks():
    # AttentionOptions::softcap and the sinks of Tensor::attend (singe/src/tensor/neural.rs:26-32,114-175; CPU meaning
    # singe/src/backend/cpu/normalization/attention.rs:250-263)
    from singe_b200 import kernel_sys as ks

    rng = np.random.default_rng(61)
    b, h, g, l, s, d = 2, 4, 2, 19, 23, 32
    q = rng.standard_normal((b, h, l, d), dtype=np.float32)
    k = rng.standard_normal((b, g, s, d), dtype=np.float32)
    v = rng.standard_normal((b, g, s, d), dtype=np.float32)
    sinks = rng.standard_normal(h).astype(np.float32)
    rep = lambda x: np.repeat(x, h // g, axis=1)
    d_q, d_k, d_v, d_sinks = dev(q), dev(k), dev(v), dev(sinks)
    out = torch.empty((b, h, l, d), device="cuda")
    stream = int(torch.cuda.current_stream().cuda_stream)
    for causal, window, softcap, with_sinks in [(True, 0, 1.5, False), (False, 0, 0.0, True), (True, 6, 0.7, True)]:
        code = ks.lib().singe_attend_f32(stream, out.data_ptr(), d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), b, h,
                                         g, l, s, d, 0.4, int(causal), window, softcap,
                                         d_sinks.data_ptr() if with_sinks else None)
        torch.cuda.synchronize()
        assert code == ks.OK
        ref = oracle.attend_options_f32(q, rep(k), rep(v), scale=0.4, causal=causal, window=window, softcap=softcap,
                                        sinks=sinks if with_sinks else None)
        assert_close_f32(host(out), ref, f"attend causal={causal} window={window} cap={softcap} sinks={with_sinks}")
    assert ks.lib().singe_attend_f32(stream, out.data_ptr(), d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), b, h, g,
                                     l, s, d, 0.4, 1, 0, -1.0, None) == ks.ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("plain_decode", [True, False])
def test_tensor_paged_attention_with_a_score_cap(plain_decode):
    # softcap on the paged surface: a plain decode batch stays on the tiled kernel (tanh.approx on the score path),
    # a mixed batch runs the general kernel; both against attend_paged with the cap
    from singe_b200 import kernel_sys as ks

    rng = np.random.default_rng(62)
    heads, kv_heads, softcap = 8, 2, 2.0
    lens = [1, 700, 16, 0, 2049, 513]
    q, kc, vc, pages, page_offsets, last = _decode_batch(rng, lens, heads, kv_heads)
    if plain_decode:
        query_offsets = np.arange(len(lens) + 1, dtype=np.int64)
    else:
        query_offsets = np.asarray([0, 1, 3, 4, 4, 5, 6], dtype=np.int64)   # sequence 1 owns two query tokens
    scale = 0.25    # large scaled scores, so the cap matters
    d_q, d_k, d_v = dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16)
    out = torch.full((len(lens), heads, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((len(lens), heads), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_qo, d_po, d_pages, d_last = dev(query_offsets), dev(page_offsets), dev(pages), dev(last)
    code = ks.lib().singe_paged_attention_options_bf16(
        int(torch.cuda.current_stream().cuda_stream), out.data_ptr(), lse.data_ptr(), d_q.data_ptr(), d_k.data_ptr(),
        d_v.data_ptr(), d_qo.data_ptr(), d_po.data_ptr(), d_pages.data_ptr(), d_last.data_ptr(), 8, len(lens), heads,
        kv_heads, 128, 16, kc.shape[0], len(lens), pages.size, scale, 1, 0, softcap, status.data_ptr())
    torch.cuda.synchronize()
    assert code == ks.OK and int(status.item()) == 0 and ops.take_device_error() == 0
    ref_code, ref_out, ref_lse = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last,
                                                         scale=scale, causal=True, softcap=softcap)
    uncapped = oracle.attend_paged_f32(q, kc, vc, query_offsets, page_offsets, pages, last, scale=scale, causal=True)[1]
    assert ref_code == oracle.OK and np.abs(uncapped - ref_out).max() > 0.1      # the cap changes the answer
    assert_close_bf16(host(out), ref_out, f"paged attention with a score cap (decode={plain_decode})")
    finite = np.isfinite(ref_lse)
    assert np.abs(host(lse)[finite] - ref_lse[finite]).max() < 5e-3


@pytest.mark.parametrize("batch,key_len,heads,kv_heads,head_dim,max_splits",
                         [(2, 300, 4, 2, 64, 4), (1, 5, 2, 1, 32, 8), (3, 1000, 8, 2, 128, 7), (2, 17, 4, 4, 16, 1)])
def test_contiguous_decode_with_split_k_and_the_fold_in_one_call(batch, key_len, heads, kv_heads, head_dim, max_splits):
    # fmha_decode_splitk_reduce_f32 (singe-kernel/src/cuda/attention/fmha.rs:1155-1241): one query per (batch, head)
    # over contiguous keys, min(max_splits, key_len) key ranges, then the fold.  The meaning is a one-token prefill
    # without a mask, which the CPU restatement of fmha_prefill_lse_f32 gives.
    from singe_b200 import kernel_sys as ks

    rng = np.random.default_rng(90 + key_len)
    q = rng.standard_normal((batch, 1, heads, head_dim), dtype=np.float32)
    k = rng.standard_normal((batch, key_len, kv_heads, head_dim), dtype=np.float32)
    v = rng.standard_normal((batch, key_len, kv_heads, head_dim), dtype=np.float32)
    scale = 1.0 / np.sqrt(head_dim)
    splits = min(max_splits, key_len)
    out = torch.full((batch, heads, head_dim), float("nan"), device="cuda")
    attn = torch.empty((batch, heads, splits, head_dim), device="cuda")
    lse = torch.empty((batch, heads, splits), device="cuda")
    d_q, d_k, d_v = dev(q), dev(k), dev(v)
    code = ks.lib().singe_fmha_decode_splitk_reduce_f32(
        int(torch.cuda.current_stream().cuda_stream), out.data_ptr(), attn.data_ptr(), lse.data_ptr(), d_q.data_ptr(),
        d_k.data_ptr(), d_v.data_ptr(), batch, key_len, heads, kv_heads, head_dim, max_splits, scale)
    torch.cuda.synchronize()
    assert code == ks.OK and ops.take_device_error() == 0
    ref_out, _ = oracle.fmha_prefill_lse_f32(q, k, v, batch=batch, query_len=1, key_len=key_len, heads=heads,
                                             kv_heads=kv_heads, head_dim=head_dim, scale=scale, causal=False)
    assert_close_f32(host(out), ref_out.reshape(batch, heads, head_dim), f"contiguous split-K decode S={key_len}")
    lib = ks.lib()
    assert lib.singe_fmha_decode_splitk_reduce_f32(None, 1, 1, 1, 1, 1, 1, 1, 8, 3, 2, 8, 0, 1.0) == ks.ERR_INVALID_LENGTH
    assert lib.singe_fmha_decode_splitk_reduce_f32(None, 1, 1, 1, 1, 1, 1, 1, 8, 4, 2, 8, 0, 1.0) == ks.ERR_INVALID_LENGTH
    assert lib.singe_fmha_decode_splitk_reduce_f32(None, None, 1, 1, 1, 1, 1, 1, 8, 4, 2, 8, 2, 1.0) == ks.ERR_NULL_POINTER
