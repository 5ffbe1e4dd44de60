"""PageTable / DecodeStep integer goldens, transcribed from the reference's own unit tests
(singe/src/nn/decode/step.rs:483-653).  Exact."""
import pytest

from singe_b200.llama import PageTable, PageTableError


def ints(a):
    return [int(x) for x in a]


def test_page_tables_give_each_sequence_its_own_pages_and_lengths():
    table = PageTable.create(2, 5, 2)
    assert table.page_count() == 7  # three pages each, and the scratch page
    step = table.step([[1, 2, 3], [4]])
    assert ints(step.tokens) == [1, 2, 3, 4]
    assert ints(step.positions) == [0, 1, 2, 0]
    assert ints(step.last_rows) == [2, 3]
    assert ints(step.query_offsets) == [0, 3, 4]
    assert ints(step.page_offsets) == [0, 2, 3]
    assert ints(step.last_page_lengths) == [1, 1]
    pages = ints(step.pages)
    assert len(pages) == 8 and pages[0] != pages[1] and pages[1] != pages[2]
    assert ints(step.write_slots) == [0, 1, 0, 0]
    assert ints(step.write_pages) == [pages[0], pages[0], pages[1], pages[2]]


def test_a_padded_step_adds_rows_that_only_padding_reads():
    table = PageTable.create(2, 5, 2).with_padding(6)
    scratch = table.scratch_page
    assert table.table_length() == 6 + 2 + 3
    step = table.step_padded([[1, 2, 3], [4]], 8)
    assert ints(step.tokens) == [1, 2, 3, 4, 0, 0, 0, 0]
    assert ints(step.positions) == [0, 1, 2, 0, 1, 2, 3, 4]
    assert ints(step.last_rows) == [2, 3]
    assert ints(step.real_tokens) == [3, 1]
    assert ints(step.sequence_ids) == [0, 0, 0, 1, 1, 1, 1, 1]
    assert ints(step.query_offsets) == [0, 3, 8]
    assert ints(step.page_offsets) == [0, 2, 5]
    assert ints(step.pages)[3:5] == [scratch, scratch]
    assert ints(step.last_page_lengths) == [1, 1]
    assert ints(step.write_pages)[4:] == [scratch] * 4
    assert ints(step.write_slots)[4:] == [1, 0, 1, 0]
    step = table.step([[5], [6]])
    assert ints(step.positions) == [3, 1]


def test_padding_stays_within_what_the_table_allows():
    table = PageTable.create(1, 8, 2).with_padding(2)
    with pytest.raises(PageTableError):
        table.step_padded([[1, 2]], 1)
    with pytest.raises(PageTableError):
        table.step_padded([[1, 2]], 5)
    step = table.step_padded([[1, 2]], 4)
    assert ints(step.last_rows) == [1] and ints(step.query_offsets) == [0, 4]


def test_page_tables_refuse_tokens_past_capacity_and_start_over_after_reset():
    table = PageTable.create(1, 2, 2)
    table.step([[1, 2]])
    with pytest.raises(PageTableError):
        table.step([[3]])
    table.reset()
    assert ints(table.step([[3]]).positions) == [0]


def test_page_tables_refuse_steps_without_a_slice_per_sequence_or_any_token():
    table = PageTable.create(2, 2, 2)
    with pytest.raises(PageTableError):
        table.step([[1]])
    with pytest.raises(PageTableError):
        table.step([[], []])


def test_a_refused_step_leaves_every_sequence_where_it_was():
    table = PageTable.create(2, 2, 2)
    table.step([[1], [2, 3]])
    with pytest.raises(PageTableError):
        table.step([[4], [5]])
    assert ints(table.step([[4], []]).positions)[0] == 1


def test_a_held_sequence_takes_one_row_and_no_capacity():
    table = PageTable.create(2, 3, 2)
    table.step([[1, 2], [3]])
    for _ in range(4):
        try:
            step = table.step([[], [4]])
        except PageTableError:
            continue
        assert ints(step.last_rows) == [0, 1]
        assert ints(step.real_tokens) == [0, 1]
        assert ints(step.positions)[0] == 2
        assert ints(step.last_page_lengths)[0] == 2
        assert ints(step.write_pages)[0] == 4
    assert ints(table.step([[9], []]).positions) == [2, 2]


def test_holding_takes_no_page():
    table = PageTable.create_shared(2, 8, 2, 4)
    table.step([[1, 2], [3]])
    assert table.free_pages() == 0
    step = table.step([[], [4]])
    assert table.free_pages() == 0 and ints(step.write_pages)[0] == 2


def test_a_released_sequence_starts_over_and_its_pages_serve_another():
    table = PageTable.create_shared(2, 8, 2, 4)
    first = table.step([[1, 2, 3], []])
    taken = ints(first.pages)[:2]
    assert table.free_pages() == 0
    with pytest.raises(PageTableError):
        table.step([[], [5]])
    table.release(0)
    assert table.free_pages() == 2
    step = table.step([[], [5]])
    assert ints(step.positions) == [0, 0]
    assert ints(step.write_pages)[1] in taken
    assert ints(step.pages)[0] == 2
    assert ints(step.page_offsets) == [0, 1, 2]
    assert ints(step.last_page_lengths) == [1, 1]
    with pytest.raises(PageTableError):
        table.release(2)


def test_a_step_that_overruns_the_pool_changes_nothing():
    table = PageTable.create_shared(2, 8, 2, 2)
    with pytest.raises(PageTableError):
        table.step([[1, 2], [3]])
    assert table.free_pages() == 1
    assert ints(table.step([[1, 2], []]).positions) == [0, 1, 0]


def test_a_full_sequence_holds_in_its_last_slot():
    table = PageTable.create(2, 2, 2)
    table.step([[1, 2], [3]])
    step = table.step([[], [4]])
    assert ints(step.positions) == [1, 1] and ints(step.last_page_lengths) == [2, 2]


def test_bulk_prompt_placement_equals_stepping_token_by_token():
    a, b = PageTable.create(3, 40, 4), PageTable.create(3, 40, 4)
    a.place_prompts([5, 0, 17])
    b.step([[1] * 5, [], [2] * 17])
    assert a.pages == b.pages and a.lengths == b.lengths and a.free == b.free


def test_decode_split_choice_fills_one_wave_when_rows_are_few():
    # 64 sequences x 2048 keys on 148 SMs (444 resident CTAs): with one KV head per rank six splits give 384 CTAs in
    # one wave; seven would start a second wave.  With all eight KV heads the rows alone fill the machine.
    from singe_b200.llama import choose_decode_splits

    one_head = choose_decode_splits(64, 2112, 512, 148)
    assert 64 * one_head <= 444 < 64 * (one_head + 2)
    assert 1 <= choose_decode_splits(512, 2112, 512, 148) <= 8
    assert choose_decode_splits(1, 16, 512, 148) == 1          # a single page cannot be split
    assert choose_decode_splits(1, 65536, 512, 148) > 8        # one long sequence alone is cut finely
