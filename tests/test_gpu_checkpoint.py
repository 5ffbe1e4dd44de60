"""A decoder built from a Hugging Face-style snapshot (config.json + safetensors, whole or in shards) computes what
the decoder built from the same weights in memory computes, alone and cut for a tensor-parallel rank."""
import json

import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import checkpoint
from singe_b200.llama import LlamaDecoder, Shard, shard_layer_weights
from tests.llama_util import MEDIUM, make_weights

pytestmark = pytest.mark.gpu

HF = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
      "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj", "attn_norm": "input_layernorm",
      "mlp_norm": "post_attention_layernorm"}


def _write_snapshot(directory, config, weights, sharded):
    fields = {"model_type": "llama", "vocab_size": config.vocab, "hidden_size": config.hidden,
              "intermediate_size": config.ffn, "num_hidden_layers": config.layers,
              "num_attention_heads": config.heads, "num_key_value_heads": config.kv_heads,
              "head_dim": config.head_dim, "rms_norm_eps": config.eps, "hidden_act": "silu",
              "rope_theta": config.theta, "tie_word_embeddings": False}
    with open(directory / "config.json", "w") as handle:
        json.dump(fields, handle)
    bits = lambda array: oracle.f32_to_bf16_bits(array).reshape(array.shape)   # the weights are bf16-representable
    tensors = {"model.embed_tokens.weight": bits(weights["embed"]), "model.norm.weight": bits(weights["final_norm"]),
               "lm_head.weight": weights["lm_head"]}                              # one tensor stored as F32: it is cast
    for index, layer in enumerate(weights["layers"]):
        for ours, theirs in HF.items():
            tensors[f"model.layers.{index}.{theirs}.weight"] = bits(layer[ours])
    if not sharded:
        checkpoint.save_safetensors(str(directory / "model.safetensors"), tensors)
        return
    names = sorted(tensors)
    weight_map = {}
    for part, members in enumerate((names[::2], names[1::2])):
        file = f"model-0000{part + 1}-of-00002.safetensors"
        checkpoint.save_safetensors(str(directory / file), {name: tensors[name] for name in members})
        weight_map.update({name: file for name in members})
    with open(directory / "model.safetensors.index.json", "w") as handle:
        json.dump({"weight_map": weight_map}, handle)


@pytest.mark.parametrize("sharded", [False, True])
def test_a_decoder_from_a_snapshot_matches_the_decoder_from_memory(tmp_path, sharded):
    config = MEDIUM
    weights = make_weights(config)
    _write_snapshot(tmp_path, config, weights, sharded)
    read_config, loaded = checkpoint.load_llama(str(tmp_path))
    assert read_config == config
    from_file = LlamaDecoder(read_config, 3, 256, weights=loaded)
    from_memory = LlamaDecoder(config, 3, 256, weights=weights)
    prompts = [[5, 9, 2, 40, 41], [7], list(range(30, 60))]
    a = from_file.step_tokens(prompts)
    b = from_memory.step_tokens(prompts)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    tokens = [[int(t)] for t in a.float().argmax(dim=1).cpu()]
    assert torch.equal(from_file.step_tokens(tokens), from_memory.step_tokens(tokens))


def test_a_rank_reads_only_its_own_rows_and_columns(tmp_path):
    # the cut a rank of two would make, without a second GPU: same tensors as shard_layer_weights cuts from memory
    config = MEDIUM
    weights = make_weights(config)
    _write_snapshot(tmp_path, config, weights, sharded=True)
    for rank in (0, 1):
        shard = Shard(rank, 2, None)
        _, loaded = checkpoint.load_llama(str(tmp_path), shard)
        for index, layer in enumerate(loaded["layers"]):
            expect = shard_layer_weights(weights["layers"][index], config, shard, interleave_gate_up=True)
            for name, tensor in layer.items():
                assert np.array_equal(tensor.float().cpu().numpy(), expect[name]), (rank, index, name)
        rows = shard.slice(config.vocab)
        assert loaded["lm_head_is_cut"] and np.array_equal(loaded["lm_head"].float().cpu().numpy(),
                                                           oracle.round_to_bf16(weights["lm_head"])[rows])
