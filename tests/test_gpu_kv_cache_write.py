"""Slot-mapped KV-cache write on the GPU against the CPU restatement: bit-exact."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops, workloads
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


def _run(cache_k, cache_v, rows_k, rows_v, pages, slots, index_dtype=np.int64):
    dk, dv = dev(cache_k), dev(cache_v)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.kv_cache_write(dk, dv, dev(rows_k), dev(rows_v), dev(np.asarray(pages, dtype=index_dtype)),
                       dev(np.asarray(slots, dtype=index_dtype)), status=status)
    torch.cuda.synchronize()
    return dk.cpu().numpy(), dv.cpu().numpy(), int(status.item())


def test_reference_cache_write_case_is_bit_exact():
    # singe/tests/nn/cache_writes.rs:43-81: f32 ramps, PAGES 4, PAGE_SIZE 4, HEADS 2, DIM 8, step [[1,2,3],[4]].
    pages, page_size, heads, dim = 4, 4, 2, 8
    count = pages * page_size * heads * dim
    ck = (np.arange(count, dtype=np.float32) + 0.5).reshape(pages, page_size, heads, dim)
    cv = (np.arange(count, dtype=np.float32) - 0.5).reshape(pages, page_size, heads, dim)
    written = (np.arange(4 * heads * dim, dtype=np.float32) + 1000.0).reshape(4, heads, dim)
    wp, ws = [0, 0, 0, 1], [0, 1, 2, 0]
    ek, ev = ck.copy(), cv.copy()
    assert oracle.kv_cache_write(ek, written, wp, ws) == oracle.OK
    assert oracle.kv_cache_write(ev, written, wp, ws) == oracle.OK
    gk, gv, status = _run(ck, cv, written, written, wp, ws)
    assert status == 0 and gk.tobytes() == ek.tobytes() and gv.tobytes() == ev.tobytes()


@pytest.mark.parametrize("index_dtype", [np.int64, np.int32])
def test_prefill_sized_write_is_bit_exact(index_dtype):
    # Config 4: 15360 tokens x 8 KV heads x 128 into 16-token pages of a permuted pool (bf16 bit patterns).
    case = workloads.prefill_case()
    rng = np.random.default_rng(3)
    total = case.total_tokens
    rows_k = rng.integers(0, 2**16, size=(total, case.kv_heads, case.head_dim), dtype=np.uint16)
    rows_v = rng.integers(0, 2**16, size=(total, case.kv_heads, case.head_dim), dtype=np.uint16)
    ck = rng.integers(0, 2**16, size=(case.pages, case.page_size, case.kv_heads, case.head_dim), dtype=np.uint16)
    cv = ck.copy()
    ek, ev = ck.copy(), cv.copy()
    assert oracle.kv_cache_write(ek, rows_k, case.write_pages, case.write_slots) == oracle.OK
    assert oracle.kv_cache_write(ev, rows_v, case.write_pages, case.write_slots) == oracle.OK
    dk = torch.from_numpy(ck.view(np.int16)).cuda().view(torch.bfloat16)
    dv = torch.from_numpy(cv.view(np.int16)).cuda().view(torch.bfloat16)
    rk = torch.from_numpy(rows_k.view(np.int16)).cuda().view(torch.bfloat16)
    rv = torch.from_numpy(rows_v.view(np.int16)).cuda().view(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.kv_cache_write(dk, dv, rk, rv, dev(case.write_pages.astype(index_dtype)),
                       dev(case.write_slots.astype(index_dtype)), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert dk.view(torch.int16).cpu().numpy().view(np.uint16).tobytes() == ek.tobytes()
    assert dv.view(torch.int16).cpu().numpy().view(np.uint16).tobytes() == ev.tobytes()
    # round trip: the rows read back through the slot map are the rows written
    flat = dk.view(torch.int16).cpu().numpy().view(np.uint16).reshape(case.pages * case.page_size, case.kv_heads,
                                                                     case.head_dim)
    back = flat[case.write_pages * case.page_size + case.write_slots]
    assert back.tobytes() == rows_k.tobytes()


def test_negative_indices_wrap_and_out_of_range_rows_are_dropped_and_reported():
    # singe/src/backend/cpu/shape/multi_index.rs:222-229
    cache = np.zeros((2, 4, 1, 4), dtype=np.float32)
    rows = (np.arange(12, dtype=np.float32) + 1).reshape(3, 1, 4)
    gk, gv, status = _run(cache, cache.copy(), rows, rows * 2, [-1, 0, 1], [-1, 0, 2])
    expect = cache.copy()
    assert oracle.kv_cache_write(expect, rows, [-1, 0, 1], [-1, 0, 2]) == oracle.OK
    assert status == 0 and gk.tobytes() == expect.tobytes() and gv.tobytes() == (expect * 2).tobytes()
    gk, gv, status = _run(cache, cache.copy(), rows, rows, [2, 0, -3], [0, 4, 0])
    assert status == 1                      # IndexOutOfBounds status word
    assert not gk.any() and not gv.any()    # every row was out of range, nothing moved


def test_large_write_through_the_bulk_copy_path_wraps_drops_and_reports():
    # 3000 tokens x K and V = 6000 rows of 512 bytes (f32, 2 heads x 64): enough rows for the kernel that stages whole
    # rows through shared memory with the bulk-copy engine.  A tenth of the indices are negative (they wrap), a
    # handful are out of range (dropped, status 1); everything else must land bit-exactly.
    rng = np.random.default_rng(21)
    pages, page_size, heads, dim, tokens = 256, 16, 2, 64, 3000
    cache_k = rng.standard_normal((pages, page_size, heads, dim), dtype=np.float32)
    cache_v = rng.standard_normal((pages, page_size, heads, dim), dtype=np.float32)
    rows_k = rng.standard_normal((tokens, heads, dim), dtype=np.float32)
    rows_v = rng.standard_normal((tokens, heads, dim), dtype=np.float32)
    slots_flat = rng.permutation(pages * page_size)[:tokens]
    write_pages = (slots_flat // page_size).astype(np.int64)
    write_slots = (slots_flat % page_size).astype(np.int64)
    wrap = rng.random(tokens) < 0.1
    write_pages[wrap] -= pages
    write_slots[wrap] -= page_size
    gk, gv, status = _run(cache_k, cache_v, rows_k, rows_v, write_pages, write_slots)
    expect_k, expect_v = cache_k.copy(), cache_v.copy()
    assert oracle.kv_cache_write(expect_k, rows_k, write_pages, write_slots) == oracle.OK
    assert oracle.kv_cache_write(expect_v, rows_v, write_pages, write_slots) == oracle.OK
    assert status == 0 and gk.tobytes() == expect_k.tobytes() and gv.tobytes() == expect_v.tobytes()
    bad_pages, bad_slots = write_pages.copy(), write_slots.copy()
    bad_pages[[5, 1700]] = pages          # one past the pool
    bad_slots[[900, 2999]] = -page_size - 1
    gk, gv, status = _run(cache_k, cache_v, rows_k, rows_v, bad_pages, bad_slots)
    assert status == 1
    keep = np.ones(tokens, dtype=bool)
    keep[[5, 1700, 900, 2999]] = False
    expect_k, expect_v = cache_k.copy(), cache_v.copy()
    assert oracle.kv_cache_write(expect_k, rows_k[keep], bad_pages[keep], bad_slots[keep]) == oracle.OK
    assert oracle.kv_cache_write(expect_v, rows_v[keep], bad_pages[keep], bad_slots[keep]) == oracle.OK
    assert gk.tobytes() == expect_k.tobytes() and gv.tobytes() == expect_v.tobytes()


def test_odd_row_width_takes_the_narrow_path():
    cache = np.zeros((3, 2, 1, 3), dtype=np.float32)   # 12-byte rows: not 16-byte vectorisable
    rows = (np.arange(6, dtype=np.float32) + 1).reshape(2, 1, 3)
    gk, gv, status = _run(cache, cache.copy(), rows, -rows, [2, 0], [1, 0])
    expect_k, expect_v = cache.copy(), cache.copy()
    oracle.kv_cache_write(expect_k, rows, [2, 0], [1, 0])
    oracle.kv_cache_write(expect_v, -rows, [2, 0], [1, 0])
    assert status == 0 and gk.tobytes() == expect_k.tobytes() and gv.tobytes() == expect_v.tobytes()
