"""The generation loop's host logic against the expectations of the reference's own unit tests
(singe/src/generation/mod.rs:769-1000: a counting decoder whose favoured token is one above the last it read)."""
import numpy as np
import pytest

from singe_b200.generation import (GeneratedToken, GenerationError, GenerationOptions, PromptChunks, RunningBatch,
                                   generate, generate_batch, step_portions)


class Counting:
    """The reference's test double (generation/mod.rs:775-830): records the steps, favours last token + 1 (mod 8)."""

    def __init__(self, sequences, largest=None):
        self._sequences = sequences
        self.largest = largest
        self.steps, self.released, self.resets = [], [], 0

    def sequences(self):
        return self._sequences

    def step(self, tokens):
        self.steps.append([list(t) for t in tokens])
        logits = np.zeros((len(tokens), 8), dtype=np.float32)
        for row, t in enumerate(tokens):
            best = (t[-1] if len(t) else 0) + 1
            logits[row, best % 8] = 1.0
        return logits

    def largest_chunk(self):
        return self.largest

    def reset(self):
        self.resets += 1

    def release(self, sequence):
        self.released.append(sequence)


def test_a_step_reads_up_to_the_largest_chunk():
    # generation/mod.rs:851-859
    assert step_portions([5, 1], None) == [5, 1]
    assert step_portions([5, 1], 3) == [4, 1]
    assert step_portions([5, 1], 8) == [5, 1]
    assert step_portions([2, 1], 0) == [1, 1]
    assert step_portions([3, 0, 3], 3) == [3, 0, 2]
    assert step_portions([1, 1], 1) == [1, 1]


def test_prompt_chunks_grow_by_four_up_to_the_capacity():
    # generation/mod.rs:861-880
    chunks = PromptChunks()
    assert chunks.sizes(512) == [16, 64, 256, 511]
    assert chunks.sizes(5000) == [16, 64, 256, 1024]
    assert chunks.sizes(10) == [9]
    assert chunks.sizes(1) == []
    assert PromptChunks.NONE.sizes(512) == []
    assert PromptChunks(16, 3).sizes(448) == [3]
    assert PromptChunks(1, 3).sizes(32) == [1, 3]


def test_a_prompt_of_any_length_reads_in_steps_up_to_the_largest_chunk():
    # generation/mod.rs:882-915
    for length in range(1, 21):
        prompt = list(range(length))
        decoder = Counting(2, largest=5)
        batch = RunningBatch.create(decoder, GenerationOptions(max_new_tokens=2))
        batch.join(prompt)
        generated = []
        while not batch.is_empty():
            generated.extend(batch.advance())
        assert len(generated) == 2
        assert generated[0].token == length % 8
        read = []
        for step in decoder.steps:
            assert sum(max(len(t), 1) for t in step) <= 7, step
            read.extend(step[0])
        assert read[:length] == prompt
        assert len(decoder.steps) == -(-length // 6) + 1   # as few steps as the largest chunk allows


def test_generation_runs_the_prompt_then_one_token_at_a_time():
    # generation/mod.rs:917-926
    decoder = Counting(1)
    seen = []
    tokens = generate(decoder, [0, 1], GenerationOptions(max_new_tokens=3), seen.append)
    assert tokens == [2, 3, 4] and seen == tokens
    assert decoder.steps == [[[0, 1]], [[2]], [[3]]]
    assert decoder.resets == 1


def test_suppressed_tokens_are_not_chosen():
    # generation/mod.rs:928-954
    decoder = Counting(1)
    options = GenerationOptions(max_new_tokens=3, suppressed_tokens=[2], first_suppressed_tokens=[1])
    assert generate(decoder, [0], options) == [0, 1, 0]
    with pytest.raises(GenerationError, match="outside a vocabulary"):
        generate(decoder, [0], GenerationOptions(max_new_tokens=1, suppressed_tokens=[8]))


def test_generation_returns_the_stop_token_and_runs_no_further():
    # generation/mod.rs:956-961
    decoder = Counting(1)
    assert generate(decoder, [0], GenerationOptions(max_new_tokens=5, stop_tokens=[2])) == [1, 2]
    assert len(decoder.steps) == 2


def test_sequences_join_and_leave_a_running_batch():
    # RunningBatch (generation/mod.rs:102-232): rows free up as sequences finish and are taken again
    decoder = Counting(2)
    batch = RunningBatch.create(decoder, GenerationOptions(max_new_tokens=2))
    assert batch.join([0]) == 0 and batch.join([3, 4]) == 1
    assert batch.join([5]) is None                        # every row is taken
    first = batch.advance()
    assert first == [GeneratedToken(0, 1, False), GeneratedToken(1, 5, False)]
    second = batch.advance()
    assert [g.finished for g in second] == [True, True] and decoder.released == [0, 1]
    assert batch.is_empty() and batch.advance() == []
    assert batch.join([6]) == 2                            # ids count the joins
    with pytest.raises(GenerationError):
        batch.join([])
    with pytest.raises(GenerationError):
        RunningBatch.create(decoder, GenerationOptions(max_new_tokens=0))


def test_generate_batch_checks_its_prompts_and_reserves_nothing_for_no_tokens():
    decoder = Counting(2)
    with pytest.raises(GenerationError):
        generate_batch(decoder, [[1]], GenerationOptions(max_new_tokens=1))          # one prompt per row
    with pytest.raises(GenerationError):
        generate_batch(decoder, [[1], []], GenerationOptions(max_new_tokens=1))
    assert generate_batch(decoder, [[1], [2]], GenerationOptions(max_new_tokens=0)) == [[], []]
    assert decoder.steps == []
    tokens = generate_batch(decoder, [[1], [2, 3, 4]], GenerationOptions(max_new_tokens=2, stop_tokens=[5]))
    assert tokens == [[2, 3], [5]]
