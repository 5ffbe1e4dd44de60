"""Pins the CPU restatement against the known-answer vectors the reference's own tests hold.

Each case cites the reference test it transcribes (file:line in tinrab/singe).
"""
import numpy as np
import pytest

from oracle import oracle


def test_sliding_window_uses_contiguous_gqa_groups():
    # singe-kernel/src/cpu/attention.rs:2234-2245
    out = oracle.sliding_window_attention_f32(
        [1.0] * 4, [1.0, 1.0], [10.0, 20.0], batch=1, query_len=1, key_len=1, heads=4, kv_heads=2, head_dim=1,
        query_start=0, key_start=0, window=1, scale=1.0, output_scale=1.0)
    assert out.tolist() == [10.0, 10.0, 20.0, 20.0]


def test_sliding_window_is_causal_left_not_symmetric():
    # singe-kernel/src/cpu/attention.rs:2247-2281
    out = oracle.sliding_window_attention_f32(
        [1.0], [1.0, 1.0, 1.0], [10.0, 20.0, 30.0], batch=1, query_len=1, key_len=3, heads=1, kv_heads=1,
        head_dim=1, query_start=1, key_start=0, window=1, scale=1.0, output_scale=1.0)
    assert out.tolist() == [20.0]


def test_readme_gemm_example():
    # singe-kernel/README.md:17-31
    out = oracle.matmul_f32([1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0], rows=2, columns=2, reduction=2,
                            lhs_row_stride=2, rhs_row_stride=2, transpose_lhs=False, transpose_rhs=False)
    assert out.tolist() == [19.0, 22.0, 43.0, 50.0]


@pytest.mark.parametrize("shape", [(0, 3, 4), (3, 0, 4), (3, 4, 0), (3, 7, 5), (17, 65, 33)])
@pytest.mark.parametrize("transpose_lhs", [False, True])
@pytest.mark.parametrize("transpose_rhs", [False, True])
def test_blocked_gemm_matches_reference_order(shape, transpose_lhs, transpose_rhs):
    # singe-kernel/tests/cpu_matmul.rs:6-86
    rows, columns, reduction = shape
    lhs = np.array([np.float32(i % 19) / np.float32(7.0) - np.float32(1.0) for i in range(rows * reduction)],
                   dtype=np.float32)
    rhs = np.array([np.float32(i % 13) / np.float32(3.0) - np.float32(2.0) for i in range(reduction * columns)],
                   dtype=np.float32)
    lhs_row = rows if transpose_lhs else reduction
    rhs_row = reduction if transpose_rhs else columns
    lhs_strides = (1, lhs_row) if transpose_lhs else (lhs_row, 1)
    rhs_strides = (1, rhs_row) if transpose_rhs else (rhs_row, 1)
    actual = np.full(rows * columns, 42.0, dtype=np.float32)
    status = oracle.matmul_strided_f32(lhs, rhs, actual, rows=rows, columns=columns, reduction=reduction,
                                       lhs_strides=lhs_strides, rhs_strides=rhs_strides)
    assert status == oracle.OK
    expected = oracle.matmul_f32(lhs, rhs, rows=rows, columns=columns, reduction=reduction, lhs_row_stride=lhs_row,
                                 rhs_row_stride=rhs_row, transpose_lhs=transpose_lhs, transpose_rhs=transpose_rhs)
    assert actual.tobytes() == expected.tobytes()


def test_blocked_gemm_checks_spans_and_supports_broadcast_strides():
    # singe-kernel/tests/cpu_matmul.rs:88-115
    output = np.zeros(4, dtype=np.float32)
    status = oracle.matmul_strided_f32([2.0, 3.0], [4.0, 5.0, 6.0, 7.0], output, rows=2, columns=2, reduction=2,
                                       lhs_strides=(0, 1), rhs_strides=(2, 1))
    assert status == oracle.OK and output.tolist() == [26.0, 31.0, 26.0, 31.0]
    assert oracle.matmul_strided_f32([1.0], [1.0], output, rows=2, columns=2, reduction=2, lhs_strides=(2, 1),
                                     rhs_strides=(2, 1)) == oracle.LENGTH_TOO_SHORT
    empty = np.zeros(0, dtype=np.float32)
    assert oracle.matmul_strided_f32(empty, empty, empty, rows=2**64 - 1, columns=2, reduction=2, lhs_strides=(2, 1),
                                     rhs_strides=(2, 1)) == oracle.SIZE_OVERFLOW
    assert oracle.matmul_strided_f32([1.0], [1.0], output, rows=2, columns=2, reduction=2,
                                     lhs_strides=(2**64 - 1, 1), rhs_strides=(2, 1)) == oracle.SIZE_OVERFLOW


# singe/tests/nn/paged_attention.rs:14-74: TOKENS 2, HEADS 2, DIM 16, SLOTS 4, PAGES 2.
TOKENS, HEADS, DIM, SLOTS, PAGES = 2, 2, 16, 4, 2
VALID = dict(query_offsets=[0, 2], page_offsets=[0, 1], pages=[0], last_page_lengths=[2])
INVALID = [
    dict(VALID, query_offsets=[0, 3]),
    dict(VALID, query_offsets=[-1, 2]),
    dict(VALID, query_offsets=[2, 0]),
    dict(VALID, page_offsets=[0, 2]),
    dict(VALID, page_offsets=[-1, 1]),
    dict(VALID, pages=[PAGES]),
    dict(VALID, pages=[-1]),
    dict(VALID, last_page_lengths=[SLOTS + 1]),
    dict(VALID, last_page_lengths=[-1]),
]


def _check(paging):
    return oracle.check_paged_values(paging["query_offsets"], paging["page_offsets"], paging["pages"],
                                     paging["last_page_lengths"], tokens=TOKENS, cache_pages=PAGES, page_size=SLOTS)


def test_paging_refusal_table():
    # singe/tests/nn/paged_attention.rs:145-184
    assert _check(VALID) == oracle.OK
    for paging in INVALID:
        assert _check(paging) == oracle.INDEX_OUT_OF_BOUNDS, paging
    assert _check(dict(VALID, last_page_lengths=[SLOTS])) == oracle.OK
    assert _check(dict(query_offsets=[0, 0], page_offsets=[0, 0], pages=[PAGES + 7],
                       last_page_lengths=[-1])) == oracle.OK


def test_attend_paged_refuses_and_accepts_like_the_reference():
    query = np.zeros((TOKENS, HEADS, DIM), dtype=np.float32)
    cache = np.zeros((PAGES, SLOTS, HEADS, DIM), dtype=np.float32)
    status, out, lse = oracle.attend_paged_f32(query, cache, cache, **VALID, scale=0.25)
    assert status == oracle.OK
    # zero scores: the first query sees one key, the second two -> lse = log2(count)
    assert np.allclose(lse[:, 0], [0.0, 1.0])
    for paging in INVALID:
        assert oracle.attend_paged_f32(query, cache, cache, **paging, scale=0.25)[0] == oracle.INDEX_OUT_OF_BOUNDS


def test_cache_write_equals_out_of_place_index_put():
    # singe/tests/nn/cache_writes.rs:43-81: PAGES 4, PAGE_SIZE 4, HEADS 2, DIM 8; ramps index + seed;
    # the step [[1,2,3],[4]] of PageTable::create(2, 8, 4) writes (page, slot) = (0,0),(0,1),(0,2),(1,0):
    # sequences take free pages in increasing order from page zero (singe/src/nn/decode/step.rs:131-132).
    pages, page_size, heads, dim = 4, 4, 2, 8
    cache = (np.arange(pages * page_size * heads * dim, dtype=np.float32) + 0.5).reshape(pages, page_size, heads, dim)
    written = (np.arange(4 * heads * dim, dtype=np.float32) + 1000.0).reshape(4, heads, dim)
    write_pages, write_slots = [0, 0, 0, 1], [0, 1, 2, 0]
    expected = cache.copy()
    for t, (p, s) in enumerate(zip(write_pages, write_slots)):
        expected[p, s] = written[t]
    assert oracle.kv_cache_write(cache, written, write_pages, write_slots) == oracle.OK
    assert cache.tobytes() == expected.tobytes()


def test_cache_write_wraps_negative_refuses_out_of_range_and_last_duplicate_wins():
    # singe/src/backend/cpu/shape/multi_index.rs:222-229 (wrap, refusal); :42-46 (last in index order wins)
    cache = np.zeros((2, 4, 3), dtype=np.float32)
    rows = np.arange(9, dtype=np.float32).reshape(3, 3) + 1
    assert oracle.kv_cache_write(cache, rows, [-1, 0, -1], [-1, 0, 3]) == oracle.OK
    assert cache[1, 3].tolist() == rows[2].tolist() and cache[0, 0].tolist() == rows[1].tolist()
    before = cache.copy()
    for bad in ([2, 0, 0], [-3, 0, 0]):
        assert oracle.kv_cache_write(cache, rows, bad, [0, 0, 0]) == oracle.INDEX_OUT_OF_BOUNDS
    assert oracle.kv_cache_write(cache, rows, [0, 0, 0], [4, 0, 0]) == oracle.INDEX_OUT_OF_BOUNDS
    assert cache.tobytes() == before.tobytes()  # a refused write moves nothing


def _paged_case(rng, batch, heads, kv_heads, head_dim, block_size, lens):
    blocks = [(n + block_size - 1) // block_size for n in lens]
    pool = sum(blocks) + 3
    perm = rng.permutation(pool)
    stride = max(max(blocks), 1) + 1
    table = np.zeros((batch, stride), dtype=np.uint32)
    at = 0
    for b, nb in enumerate(blocks):
        table[b, :nb] = perm[at:at + nb]
        at += nb
    k = rng.standard_normal((pool, block_size, kv_heads, head_dim)).astype(np.float32)
    v = rng.standard_normal((pool, block_size, kv_heads, head_dim)).astype(np.float32)
    q = rng.standard_normal((batch, heads, head_dim)).astype(np.float32)
    return q, k, v, table, stride


def test_decode_matches_float64_softmax_and_gathers_through_the_block_table():
    rng = np.random.default_rng(7)
    batch, heads, kv_heads, head_dim, block_size = 3, 4, 2, 8, 4
    lens = [5, 0, 11]
    q, k, v, table, stride = _paged_case(rng, batch, heads, kv_heads, head_dim, block_size, lens)
    scale = 1.0 / np.sqrt(head_dim)
    out = oracle.paged_kv_decode_attention_f32(q, k, v, lens, table, batch=batch, heads=heads, kv_heads=kv_heads,
                                               head_dim=head_dim, block_size=block_size,
                                               block_table_batch_stride=stride, scale=scale)
    for b in range(batch):
        for h in range(heads):
            g = h // (heads // kv_heads)
            if lens[b] == 0:
                assert not out[b, h].any()
                continue
            keys = np.stack([k[table[b, i // block_size], i % block_size, g] for i in range(lens[b])]).astype(np.float64)
            vals = np.stack([v[table[b, i // block_size], i % block_size, g] for i in range(lens[b])]).astype(np.float64)
            s = keys @ q[b, h].astype(np.float64) * scale
            p = np.exp(s - s.max())
            p /= p.sum()
            assert np.abs(out[b, h] - p @ vals).max() < 1e-5


def test_split_partials_reduce_to_the_unsplit_decode():
    # Partials as the split-K decode defines them (singe-kernel/src/cuda/attention/mod.rs:2456-2509):
    # split s covers keys [s*ceil(L/splits), ...), partial = softmax within the split . V, lse = max + ln(sum).
    rng = np.random.default_rng(8)
    batch, heads, kv_heads, head_dim, block_size, splits = 2, 4, 2, 8, 4, 3
    lens = [12, 12]
    q, k, v, table, stride = _paged_case(rng, batch, heads, kv_heads, head_dim, block_size, lens)
    scale = 0.3
    full = oracle.paged_kv_decode_attention_f32(q, k, v, lens, table, batch=batch, heads=heads, kv_heads=kv_heads,
                                                head_dim=head_dim, block_size=block_size,
                                                block_table_batch_stride=stride, scale=scale)
    per = 4
    attn = np.zeros((batch, heads, splits, head_dim), dtype=np.float32)
    lse = np.zeros((batch, heads, splits), dtype=np.float32)
    for b in range(batch):
        for h in range(heads):
            g = h // 2
            for s in range(splits):
                idx = range(s * per, (s + 1) * per)
                keys = np.stack([k[table[b, i // block_size], i % block_size, g] for i in idx]).astype(np.float64)
                vals = np.stack([v[table[b, i // block_size], i % block_size, g] for i in idx]).astype(np.float64)
                sc = keys @ q[b, h].astype(np.float64) * scale
                p = np.exp(sc - sc.max())
                lse[b, h, s] = sc.max() + np.log(p.sum())
                attn[b, h, s] = (p / p.sum()) @ vals
    reduced = oracle.splitk_reduce_f32(attn, lse, batch=batch, heads=heads, splits=splits, head_dim=head_dim)
    assert np.abs(reduced - full).max() < 1e-5


def test_packed_prefill_surfaces_agree_where_their_causal_rules_coincide():
    # len_q == len_kv: sequence-local causal (singe-kernel) == queries-as-last-tokens (Tensor surface).
    rng = np.random.default_rng(9)
    heads, kv_heads, head_dim, block_size = 4, 2, 8, 4
    lens = [6, 3]
    offsets = [0, 6]
    total = sum(lens)
    q = rng.standard_normal((total, heads, head_dim)).astype(np.float32)
    kr = rng.standard_normal((total, kv_heads, head_dim)).astype(np.float32)
    vr = rng.standard_normal((total, kv_heads, head_dim)).astype(np.float32)
    scale = 1.0 / np.sqrt(head_dim)
    out_r, lse_r = oracle.ragged_kv_prefill_attention_f32(q, kr, vr, lens, lens, offsets, batch=2,
                                                          total_query_tokens=total, heads=heads, kv_heads=kv_heads,
                                                          head_dim=head_dim, causal=True, scale=scale)
    # the same keys placed in pages
    blocks = [2, 1]
    pool = 5
    perm = rng.permutation(pool)
    table = np.zeros((2, 3), dtype=np.uint32)
    table[0, :2] = perm[:2]
    table[1, :1] = perm[2:3]
    kc = np.zeros((pool, block_size, kv_heads, head_dim), dtype=np.float32)
    vc = np.zeros_like(kc)
    wp, ws = [], []
    for b in range(2):
        for i in range(lens[b]):
            wp.append(int(table[b, i // block_size]))
            ws.append(i % block_size)
    assert oracle.kv_cache_write(kc, kr, wp, ws) == oracle.OK
    assert oracle.kv_cache_write(vc, vr, wp, ws) == oracle.OK
    out_p, lse_p = oracle.paged_kv_prefill_attention_f32(q, kc, vc, lens, lens, offsets, table, batch=2,
                                                         total_query_tokens=total, heads=heads, kv_heads=kv_heads,
                                                         head_dim=head_dim, block_size=block_size,
                                                         block_table_batch_stride=3, causal=True, scale=scale)
    assert out_p.tobytes() == out_r.tobytes() and lse_p.tobytes() == lse_r.tobytes()
    status, out_t, lse_t = oracle.attend_paged_f32(
        q, kc, vc, [0, 6, 9], [0, 2, 3], [int(table[0, 0]), int(table[0, 1]), int(table[1, 0])], [2, 3], scale=scale)
    assert status == oracle.OK
    assert np.abs(out_t - out_r).max() < 1e-6
    assert np.abs(lse_t * np.log(2.0) - lse_r).max() < 1e-5  # base 2 vs natural log


def test_dense_prefill_and_tensor_sdpa_agree():
    rng = np.random.default_rng(10)
    b, h, g, l, d = 1, 4, 2, 9, 8
    q = rng.standard_normal((b, l, h, d)).astype(np.float32)
    k = rng.standard_normal((b, l, g, d)).astype(np.float32)
    v = rng.standard_normal((b, l, g, d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    out, lse = oracle.fmha_prefill_lse_f32(q, k, v, batch=b, query_len=l, key_len=l, heads=h, kv_heads=g,
                                           head_dim=d, scale=scale, causal=True)
    rep = h // g
    qt = q.transpose(0, 2, 1, 3)
    kt = np.repeat(k.transpose(0, 2, 1, 3), rep, axis=1)
    vt = np.repeat(v.transpose(0, 2, 1, 3), rep, axis=1)
    dense = oracle.scaled_dot_product_attention_f32(qt, kt, vt, scale=scale, causal=True)
    assert dense.transpose(0, 2, 1, 3).tobytes() == out.tobytes()


def test_bf16_rounding_is_nearest_even():
    values = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 0.0], dtype=np.float32)
    bits = oracle.f32_to_bf16_bits(values)
    # 1.00390625 = 0x3F808000 is a tie -> even mantissa (0x3F80); 1.01171875 = 0x3F818000 ties up to 0x3F82.
    assert bits.tolist()[:3] == [0x3F80, 0x3F80, 0x3F82]
    assert oracle.round_to_bf16(values).tolist()[:3] == [1.0, 1.0, 1.015625]
    torch = pytest.importorskip("torch")
    rnd = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    expect = torch.from_numpy(rnd).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (oracle.f32_to_bf16_bits(rnd) == expect).all()


def test_linear_bf16_rounds_once():
    rng = np.random.default_rng(2)
    m, n, k = 3, 5, 64
    x = oracle.f32_to_bf16_bits(rng.standard_normal((m, k)).astype(np.float32))
    w = oracle.f32_to_bf16_bits((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    wide = oracle.linear_bf16_f32(x, w, m=m, n=n, k=k)
    narrow = oracle.linear_bf16(x, w, m=m, n=n, k=k)
    assert (oracle.f32_to_bf16_bits(wide) == narrow).all()
    ref = oracle.bf16_bits_to_f32(x).astype(np.float64) @ oracle.bf16_bits_to_f32(w).astype(np.float64).T
    assert np.abs(wide - ref).max() < 1e-4
