"""The Llama-shaped decode step on the GPU against the CPU restatement of the reference's eager bf16 path."""
import numpy as np
import pytest
import torch

from oracle import llama_ref
from singe_b200.llama import LlamaDecoder, PageTable, rotary_tables
from tests.gpu_util import assert_close_bf16, host
from tests.llama_util import MEDIUM, TINY, make_context, make_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("config,context", [(TINY, [3, 9, 0, 17]), (MEDIUM, [40, 0, 129, 16, 700])])
@pytest.mark.parametrize("graph", [False, True])
def test_decode_steps_match_the_reference_path(config, context, graph):
    sequences, capacity = len(context), 768
    weights = make_weights(config)
    decoder = LlamaDecoder(config, sequences, capacity, weights=weights)
    keys, values = make_context(config, decoder.table.page_count())
    for layer in range(config.layers):
        decoder.key_caches[layer].copy_(torch.from_numpy(keys[layer]).to(torch.bfloat16))
        decoder.value_caches[layer].copy_(torch.from_numpy(values[layer]).to(torch.bfloat16))
    decoder.table.place_prompts(context)
    reference_table = PageTable.create(sequences, capacity, config.page_size)
    reference_table.place_prompts(context)
    cos, sin = rotary_tables(config.head_dim, config.theta, capacity)
    if graph:
        decoder.plan([1] * sequences)      # any valid step gives the capture its shapes
        decoder.table = PageTable.create(sequences, capacity, config.page_size)
        decoder.table.place_prompts(context)
        decoder.capture()
        for layer in range(config.layers):  # the warm-up and capture runs wrote into the caches: restore them
            decoder.key_caches[layer].copy_(torch.from_numpy(keys[layer]).to(torch.bfloat16))
            decoder.value_caches[layer].copy_(torch.from_numpy(values[layer]).to(torch.bfloat16))
    rng = np.random.default_rng(11)
    for _ in range(3):
        tokens = rng.integers(0, config.vocab, size=sequences)
        step = reference_table.step([[int(t)] for t in tokens])
        expect = llama_ref.decode_step(config, weights, keys, values, step, cos, sin)
        next_tokens = decoder.step(tokens)
        torch.cuda.synchronize()
        assert int(decoder.status.item()) == 0
        assert_close_bf16(host(decoder.logits), expect, f"logits ({'graph' if graph else 'eager'})")
        for layer in range(config.layers):  # rotated keys and values landed in the same cache slots
            assert_close_bf16(host(decoder.key_caches[layer]), keys[layer], f"key cache {layer}")
            assert_close_bf16(host(decoder.value_caches[layer]), values[layer], f"value cache {layer}")
        # greedy token: equal to the oracle's argmax unless the two best logits are within tolerance of each other
        top = np.sort(expect, axis=1)[:, -2:]
        clear = (top[:, 1] - top[:, 0]) > 0.05
        assert (host(next_tokens).astype(np.int64)[clear] == expect.argmax(axis=1)[clear]).all()


def test_one_layer_at_the_full_llama3_8b_width_and_batch():
    # Config 5's layer shape (hidden 4096, 32 Q / 8 KV heads of 128, SwiGLU 14336, 64 sequences near context 2048) with a
    # single layer and a small vocabulary: the split-K GEMMs, the SwiGLU epilogue at N = 28672, the one-wave decode
    # splits and the 4096-wide glue kernels all run at their benchmark sizes against the CPU restatement.
    from singe_b200.llama import LlamaConfig

    config = LlamaConfig(layers=1, vocab=2048)
    sequences, capacity = 64, 2048 + 64
    context = [2048 - 37 * (i % 5) for i in range(sequences)]
    weights = make_weights(config)
    decoder = LlamaDecoder(config, sequences, capacity, weights=weights)
    keys, values = make_context(config, decoder.table.page_count())
    decoder.key_caches[0].copy_(torch.from_numpy(keys[0]).to(torch.bfloat16))
    decoder.value_caches[0].copy_(torch.from_numpy(values[0]).to(torch.bfloat16))
    decoder.table.place_prompts(context)
    reference_table = PageTable.create(sequences, capacity, config.page_size)
    reference_table.place_prompts(context)
    cos, sin = rotary_tables(config.head_dim, config.theta, capacity)
    tokens = np.random.default_rng(4).integers(0, config.vocab, size=sequences)
    step = reference_table.step([[int(t)] for t in tokens])
    expect = llama_ref.decode_step(config, weights, keys, values, step, cos, sin)
    decoder.step(tokens)
    torch.cuda.synchronize()
    assert int(decoder.status.item()) == 0
    assert_close_bf16(host(decoder.logits), expect, "logits at full width")
    assert_close_bf16(host(decoder.key_caches[0]), keys[0], "key cache at full width")
