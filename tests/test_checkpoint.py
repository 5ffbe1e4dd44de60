"""The checkpoint path's host side: config.json parsing, the safetensors reader against the safetensors library,
sharded indexes, key and shape checks.  (The device side -- a decoder built from a snapshot -- is in
tests/test_gpu_checkpoint.py.)"""
import json
import os

import numpy as np
import pytest

from singe_b200 import checkpoint
from singe_b200.llama import LlamaConfig

CONFIG = {"model_type": "llama", "vocab_size": 97, "hidden_size": 64, "intermediate_size": 128,
          "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-5,
          "hidden_act": "silu", "rope_theta": 500000.0, "tie_word_embeddings": False}


def _write_config(directory, **changes):
    fields = dict(CONFIG, **changes)
    fields = {k: v for k, v in fields.items() if v is not None}
    with open(os.path.join(directory, "config.json"), "w") as handle:
        json.dump(fields, handle)


def _tensors(config: LlamaConfig, tied=False, seed=0):
    rng = np.random.default_rng(seed)
    return {name: rng.standard_normal(shape, dtype=np.float32) * np.float32(0.05)
            for name, shape in checkpoint.llama_names(config, tied).items()}


def test_config_fields_and_defaults(tmp_path):
    _write_config(tmp_path)
    config = checkpoint.read_config(str(tmp_path))
    assert config == LlamaConfig(layers=2, hidden=64, heads=4, kv_heads=2, head_dim=16, ffn=128, vocab=97, eps=1e-5,
                                 theta=500000.0)
    _write_config(tmp_path, num_key_value_heads=None, head_dim=32, rope_theta=None)
    config = checkpoint.read_config(str(tmp_path))
    assert (config.kv_heads, config.head_dim, config.theta) == (4, 32, 10000.0)   # singe-model/src/config.rs:117-121


@pytest.mark.parametrize("changes,what", [
    ({"layer_types": ["full_attention", "sliding_attention"]}, "full attention"),   # config.rs:142-153
    ({"attention_bias": True}, "biases"),
    ({"hidden_act": "gelu"}, "activation"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "rotary type llama3"),
])
def test_configs_the_decoder_would_compute_wrongly_are_refused(tmp_path, changes, what):
    _write_config(tmp_path, **changes)
    with pytest.raises(checkpoint.UnsupportedConfig, match=what):
        checkpoint.read_config(str(tmp_path))


def test_reader_and_writer_agree_with_the_safetensors_library(tmp_path):
    safetensors_numpy = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(1)
    tensors = {"a.weight": rng.standard_normal((5, 7), dtype=np.float32),
               "b": rng.standard_normal((3,), dtype=np.float32).astype(np.float16),
               "c.bits": rng.integers(0, 1 << 16, size=(4, 2, 3), dtype=np.uint16)}
    # written by the library (bf16 has no numpy type: written through F16/F32 only), read here
    library_file = str(tmp_path / "library.safetensors")
    safetensors_numpy.save_file({k: v for k, v in tensors.items() if v.dtype != np.uint16}, library_file)
    ours = checkpoint.SafetensorsFile(library_file)
    assert sorted(ours.names()) == ["a.weight", "b"]
    assert np.array_equal(ours.array("a.weight"), tensors["a.weight"]) and ours.dtype("b") == "F16"
    assert np.array_equal(ours.array("a.weight")[1:3], tensors["a.weight"][1:3])       # a partial read is a view
    # written here, read by the library
    our_file = str(tmp_path / "ours.safetensors")
    checkpoint.save_safetensors(our_file, {k: v for k, v in tensors.items() if v.dtype != np.uint16})
    back = safetensors_numpy.load_file(our_file)
    assert all(np.array_equal(back[k], tensors[k]) for k in back) and sorted(back) == ["a.weight", "b"]
    # bf16 bit patterns survive a round trip through our writer and reader
    checkpoint.save_safetensors(our_file, tensors)
    again = checkpoint.SafetensorsFile(our_file)
    assert again.dtype("c.bits") == "BF16" and np.array_equal(again.array("c.bits"), tensors["c.bits"])


def test_malformed_files_are_refused(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\x10")
    with pytest.raises(checkpoint.CheckpointError, match="too short"):
        checkpoint.SafetensorsFile(str(path))
    path.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(checkpoint.CheckpointError, match="exceeds"):
        checkpoint.SafetensorsFile(str(path))
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    path.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(checkpoint.CheckpointError, match="offsets"):
        checkpoint.SafetensorsFile(str(path))


def test_missing_unexpected_and_misshapen_tensors_are_errors(tmp_path):
    config = checkpoint.read_config(_snapshot(tmp_path, CONFIG))
    expected = checkpoint.llama_names(config, tied=False)
    tensors = _tensors(config)
    checkpoint.save_safetensors(str(tmp_path / "model.safetensors"), tensors)
    checkpoint.check_keys(checkpoint.Snapshot(str(tmp_path)), expected)                 # complete: accepted
    extra = dict(tensors, **{"model.layers.0.self_attn.rotary_emb.inv_freq": np.zeros(8, dtype=np.float32)})
    checkpoint.save_safetensors(str(tmp_path / "model.safetensors"), extra)
    checkpoint.check_keys(checkpoint.Snapshot(str(tmp_path)), expected)                 # old rotary buffer: ignored
    broken = {k: v for k, v in tensors.items() if k != "model.norm.weight"}
    broken["model.layers.7.mlp.up_proj.weight"] = np.zeros((2, 2), dtype=np.float32)
    checkpoint.save_safetensors(str(tmp_path / "model.safetensors"), broken)
    with pytest.raises(checkpoint.CheckpointError, match=r"missing \['model.norm.weight'\].*unexpected \['model.layers.7"):
        checkpoint.check_keys(checkpoint.Snapshot(str(tmp_path)), expected)
    wrong = dict(tensors, **{"model.norm.weight": np.zeros(3, dtype=np.float32)})
    checkpoint.save_safetensors(str(tmp_path / "model.safetensors"), wrong)
    with pytest.raises(checkpoint.CheckpointError, match="shape"):
        checkpoint.check_keys(checkpoint.Snapshot(str(tmp_path)), expected)


def test_a_sharded_checkpoint_is_found_through_its_index(tmp_path):
    config = checkpoint.read_config(_snapshot(tmp_path, CONFIG))
    tensors = _tensors(config)
    names = sorted(tensors)
    halves = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    weight_map = {}
    for file, members in halves.items():
        checkpoint.save_safetensors(str(tmp_path / file), {name: tensors[name] for name in members})
        weight_map.update({name: file for name in members})
    with open(tmp_path / "model.safetensors.index.json", "w") as handle:
        json.dump({"metadata": {}, "weight_map": weight_map}, handle)
    snapshot = checkpoint.Snapshot(str(tmp_path))
    checkpoint.check_keys(snapshot, checkpoint.llama_names(config, tied=False))
    assert all(np.array_equal(snapshot.array(name), tensors[name]) for name in names)
    weight_map["model.norm.weight"] = "model-00001-of-00002.safetensors" if "model.norm.weight" in halves[
        "model-00002-of-00002.safetensors"] else "model-00002-of-00002.safetensors"
    with open(tmp_path / "model.safetensors.index.json", "w") as handle:
        json.dump({"weight_map": weight_map}, handle)
    with pytest.raises(checkpoint.CheckpointError, match="does not hold"):
        checkpoint.Snapshot(str(tmp_path)).array("model.norm.weight")


def _snapshot(tmp_path, fields):
    _write_config(tmp_path, **{k: v for k, v in fields.items() if k not in CONFIG})
    return str(tmp_path)
