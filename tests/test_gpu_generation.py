"""Prompt steps and the generation loop on the GPU against the CPU restatement of the reference's eager path.

A prompt goes through the same kernels a serving loop would chain: embedding, QKV GEMM at M = prompt tokens, rotary +
slot-mapped cache write, the packed causal prefill kernel over the cache just written, o_proj / SwiGLU MLP, logits of
each sequence's last token; then decode steps read the cache the prompt step filled."""
import numpy as np
import pytest
import torch

from oracle import llama_ref
from singe_b200.generation import GenerationOptions, RunningBatch, generate_batch
from singe_b200.llama import CachedDecoder, LlamaDecoder, PageTable, PageTableError, rotary_tables
from tests.gpu_util import assert_close_bf16, host
from tests.llama_util import MEDIUM, TINY, make_weights

pytestmark = pytest.mark.gpu


class Reference:
    """The CPU side: its own page table and float32 caches, stepped with the same token lists."""

    def __init__(self, config, sequences, capacity, weights):
        self.config, self.weights = config, weights
        self.table = PageTable.create(sequences, capacity, config.page_size)
        shape = (self.table.page_count(), config.page_size, config.kv_heads, config.head_dim)
        self.keys = [np.zeros(shape, dtype=np.float32) for _ in range(config.layers)]
        self.values = [np.zeros(shape, dtype=np.float32) for _ in range(config.layers)]
        self.cos, self.sin = rotary_tables(config.head_dim, config.theta, capacity)

    def step(self, tokens):
        step = self.table.step(tokens)
        return llama_ref.decode_step(self.config, self.weights, self.keys, self.values, step, self.cos, self.sin)


def _check_step(decoder, reference, tokens, what):
    logits = decoder.step_tokens(tokens)
    torch.cuda.synchronize()
    assert int(decoder.status.item()) == 0
    expect = reference.step(tokens)
    live = [row for row, t in enumerate(tokens) if len(t) > 0]   # an idle row's logits mean nothing
    assert_close_bf16(host(logits)[live], expect[live], f"{what}: logits")
    pool = decoder.table.pool   # the scratch page behind the pool holds whatever idle rows wrote
    for layer in range(decoder.config.layers):
        assert_close_bf16(host(decoder.key_caches[layer])[:pool], reference.keys[layer][:pool], f"{what}: key cache")
        assert_close_bf16(host(decoder.value_caches[layer])[:pool], reference.values[layer][:pool], f"{what}: values")
    return host(logits), expect


@pytest.mark.parametrize("config,prompts", [
    (TINY, [[5, 6, 7], [1], [9, 8, 7, 6, 5, 4, 3, 2, 1], list(range(20, 37))]),
    # head_dim 128, 16-token pages: the tcgen05 prefill kernel; lengths cross page (16) and query-tile (128, 256) edges
    (MEDIUM, [list(range(1, 131)), [3] * 16, list(range(100, 400)), [7]]),
])
def test_prompt_then_chunk_then_decode_steps_match_the_reference_path(config, prompts):
    sequences, capacity = len(prompts), 768
    weights = make_weights(config)
    decoder = LlamaDecoder(config, sequences, capacity, weights=weights)
    reference = Reference(config, sequences, capacity, weights)
    rng = np.random.default_rng(21)
    prompts = [[int(t) % config.vocab for t in p] for p in prompts]
    _check_step(decoder, reference, prompts, "prompt step")
    # a second chunk behind the context just cached (queries are the LAST tokens of longer sequences), one row idle
    more = [[int(t) for t in rng.integers(0, config.vocab, size=n)] for n in (40, 0, 3, 130)]
    _check_step(decoder, reference, more, "chunk behind a context")
    # then plain decode steps over everything cached so far
    for index in range(2):
        tokens = [[int(t)] for t in rng.integers(0, config.vocab, size=sequences)]
        got, expect = _check_step(decoder, reference, tokens, f"decode step {index}")
        top = np.sort(expect, axis=1)[:, -2:]
        clear = (top[:, 1] - top[:, 0]) > 0.05
        assert (got.argmax(axis=1)[clear] == expect.argmax(axis=1)[clear]).all()


def test_a_step_that_overruns_the_cache_changes_nothing():
    config = TINY
    decoder = LlamaDecoder(config, 2, 16, weights=make_weights(config))
    decoder.step_tokens([[1, 2, 3], [4]])
    lengths = list(decoder.table.lengths)
    with pytest.raises(PageTableError):
        decoder.step_tokens([list(range(20)), [5]])        # 3 + 20 tokens pass the capacity of 16
    assert decoder.table.lengths == lengths
    decoder.step_tokens([[6], [7]])                        # and the decoder still steps
    torch.cuda.synchronize()
    assert int(decoder.status.item()) == 0


def test_generation_over_the_gpu_decoder_follows_the_reference_path_token_by_token():
    # Continuous batching through RunningBatch: three prompts over two rows, so the third joins when a row frees up.
    # Every step's logits are compared with the CPU restatement fed the same tokens (the GPU's choices).
    config = TINY
    weights = make_weights(config)
    model = LlamaDecoder(config, 2, 64, weights=weights)
    reference = Reference(config, 2, 64, weights)

    class Checked(CachedDecoder):
        def step(self, tokens):
            logits = super().step(tokens)
            torch.cuda.synchronize()
            expect = reference.step([list(t) for t in tokens])
            live = [row for row, t in enumerate(tokens) if len(t) > 0]
            assert_close_bf16(host(logits)[live], expect[live], "generation step logits")
            return logits

        def reset(self):
            super().reset()
            reference.table.reset()

        def release(self, sequence):
            super().release(sequence)
            reference.table.release(sequence)

    decoder = Checked(model)
    assert decoder.largest_chunk() == 63 and decoder.sequences() == 2
    batch = RunningBatch.create(decoder, GenerationOptions(max_new_tokens=4))
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [2, 7], [1, 8, 2, 8, 1, 8]]
    waiting = list(prompts)
    outputs = {}
    while waiting or not batch.is_empty():
        while waiting and batch.join(waiting[0]) is not None:
            waiting.pop(0)
        for generated in batch.advance():
            outputs.setdefault(generated.sequence, []).append(generated.token)
    assert sorted(outputs) == [0, 1, 2] and all(len(tokens) == 4 for tokens in outputs.values())
    assert model.table.free_pages() == model.table.pool    # every sequence released its pages
    # the batch helper gives the same tokens for the first two prompts run together
    again = generate_batch(Checked(model), prompts[:2], GenerationOptions(max_new_tokens=4))
    assert again == [outputs[0], outputs[1]]
