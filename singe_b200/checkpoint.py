"""Hugging Face snapshot -> decoder configuration -> this rank's weight shards, read straight out of safetensors.

Mirrors the reference's checkpoint path for the Llama shape:
  ``DecoderConfig`` / ``Snapshot::config``   singe-model/src/config.rs:110-176,186-214 (``config.json`` fields, defaults for
                                             ``num_key_value_heads`` and ``head_dim``, refusal of sliding layers)
  ``llama::load``                            singe-model/src/text/text_generation/llama/mod.rs:17-22
  ``load_weights`` / ``load_checkpoint``     singe-model/src/assembly/weights.rs:14-29, singe/src/nn/checkpoint.rs:95-137
                                             (``model.safetensors`` or the shards ``model.safetensors.index.json`` names)
  ``check_keys``                             singe/src/nn/checkpoint.rs:140-190 (missing and unexpected names are errors)
  ``safetensors_bytes``                      singe/src/nn/checkpoint.rs:36-60 (``save_safetensors`` here)
What is new is the tensor-parallel cut: a rank memory-maps the files and copies only its rows (q/k/v, gate/up, LM
head) or columns (o_proj, down_proj) to the device, so no rank ever holds the whole model.

The safetensors layout is read directly (8-byte little-endian header length, a JSON header of
``{name: {dtype, shape, data_offsets}}``, then the raw little-endian tensor bytes), which is what makes the partial
reads possible.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

from .llama import LlamaConfig, Shard

CHECKPOINT_STEMS = ("model", "diffusion_pytorch_model")   # transformers' name first, then diffusers'

_DTYPES = {"BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4)}


class CheckpointError(ValueError):
    pass


class UnsupportedConfig(ValueError):
    pass


# ------------------------------------------------------------------------------------------------
# config.json
# ------------------------------------------------------------------------------------------------

def read_config(snapshot: str) -> LlamaConfig:
    """``config.json`` of a Llama-family snapshot as a ``LlamaConfig``.  Refuses what the decoder here would compute
    wrongly instead of ignoring it: sliding-window layers, projection biases, an activation other than SiLU, scaled
    rotary frequencies, a partial rotary dimension."""
    with open(os.path.join(snapshot, "config.json")) as handle:
        fields = json.load(handle)
    need = lambda name: fields[name] if name in fields else _missing(name)
    heads = int(need("num_attention_heads"))
    hidden = int(need("hidden_size"))
    if any(layer != "full_attention" for layer in fields.get("layer_types") or []):
        raise UnsupportedConfig("a layer other than full attention")
    if fields.get("attention_bias") or fields.get("mlp_bias"):
        raise UnsupportedConfig("projection biases")
    activation = fields.get("hidden_act", fields.get("hidden_activation"))
    if activation not in ("silu", "swish"):
        raise UnsupportedConfig(f"activation {activation}")
    scaling = fields.get("rope_scaling")
    if scaling and (scaling.get("rope_type") or scaling.get("type") or "default") != "default":
        raise UnsupportedConfig(f"rotary type {scaling.get('rope_type') or scaling.get('type')}")
    if float(fields.get("partial_rotary_factor", 1.0)) != 1.0:
        raise UnsupportedConfig("a partial rotary dimension")
    return LlamaConfig(layers=int(need("num_hidden_layers")), hidden=hidden, heads=heads,
                       kv_heads=int(fields.get("num_key_value_heads") or heads),
                       head_dim=int(fields.get("head_dim") or hidden // heads), ffn=int(need("intermediate_size")),
                       vocab=int(need("vocab_size")), eps=float(need("rms_norm_eps")),
                       theta=float(fields.get("rope_theta", 10000.0)))


def tied_embeddings(snapshot: str) -> bool:
    with open(os.path.join(snapshot, "config.json")) as handle:
        return bool(json.load(handle).get("tie_word_embeddings") or False)


def _missing(name):
    raise UnsupportedConfig(f"config.json has no {name}")


# ------------------------------------------------------------------------------------------------
# safetensors files
# ------------------------------------------------------------------------------------------------

class SafetensorsFile:
    """One file, memory-mapped; ``rows``/``columns`` return views of a tensor's bytes without reading the rest."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as handle:
            prefix = handle.read(8)
            if len(prefix) != 8:
                raise CheckpointError(f"{path}: too short for a safetensors header")
            (length,) = struct.unpack("<Q", prefix)
            if length > os.path.getsize(path) - 8:
                raise CheckpointError(f"{path}: header length {length} exceeds the file")
            header = json.loads(handle.read(length))
        self.entries = {name: entry for name, entry in header.items() if name != "__metadata__"}
        self.data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + length)
        for name, entry in self.entries.items():
            begin, end = entry["data_offsets"]
            if entry["dtype"] not in _DTYPES:
                raise CheckpointError(f"{path}: {name} has unsupported dtype {entry['dtype']}")
            count = int(np.prod(entry["shape"], dtype=np.int64)) if entry["shape"] else 1
            if end - begin != count * _DTYPES[entry["dtype"]][1] or end > self.data.size:
                raise CheckpointError(f"{path}: {name} has data offsets that do not match its shape")

    def names(self):
        return list(self.entries)

    def array(self, name: str) -> np.ndarray:
        entry = self.entries[name]
        begin, end = entry["data_offsets"]
        dtype, _ = _DTYPES[entry["dtype"]]
        return self.data[begin:end].view(dtype).reshape(entry["shape"])

    def dtype(self, name: str) -> str:
        return self.entries[name]["dtype"]


def save_safetensors(path: str, tensors: dict) -> None:
    """Writes ``{name: array}`` (float32 / float16 arrays, or uint16 arrays holding bf16 bit patterns) as one
    safetensors file, names sorted, replacing ``path``."""
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        array = np.ascontiguousarray(tensors[name])
        kind = {np.dtype(np.uint16): "BF16", np.dtype(np.float16): "F16", np.dtype(np.float32): "F32"}.get(array.dtype)
        if kind is None:
            raise CheckpointError(f"{name}: unsupported checkpoint data type {array.dtype}")
        blob = array.tobytes()
        header[name] = {"dtype": kind, "shape": list(array.shape), "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for blob in blobs:
            handle.write(blob)


class Snapshot:
    """The checkpoint of a snapshot directory: ``model.safetensors``, or the shards its index names."""

    def __init__(self, directory: str):
        self.directory = directory
        stem = next((s for s in CHECKPOINT_STEMS
                     if os.path.exists(os.path.join(directory, f"{s}.safetensors"))
                     or os.path.exists(os.path.join(directory, f"{s}.safetensors.index.json"))), CHECKPOINT_STEMS[0])
        index = os.path.join(directory, f"{stem}.safetensors.index.json")
        self.files = {}
        if os.path.exists(index):
            with open(index) as handle:
                try:
                    self.where = dict(json.load(handle)["weight_map"])
                except (KeyError, ValueError) as error:
                    raise CheckpointError(f"{index}: {error}") from error
        else:
            single = f"{stem}.safetensors"
            if not os.path.exists(os.path.join(directory, single)):
                raise CheckpointError(f"{directory} holds no {single} and no index of shards")
            self.where = {name: single for name in self._file(single).names()}

    def _file(self, name: str) -> SafetensorsFile:
        if name not in self.files:
            self.files[name] = SafetensorsFile(os.path.join(self.directory, name))
        return self.files[name]

    def names(self):
        return list(self.where)

    def array(self, name: str) -> np.ndarray:
        source = self._file(self.where[name])
        if name not in source.entries:
            raise CheckpointError(f"{self.where[name]} does not hold {name}, which the index says it does")
        return source.array(name)

    def dtype(self, name: str) -> str:
        return self._file(self.where[name]).dtype(name)


# ------------------------------------------------------------------------------------------------
# Llama weights, cut for one rank
# ------------------------------------------------------------------------------------------------

def llama_names(config: LlamaConfig, tied: bool) -> dict:
    """Hugging Face parameter name -> expected shape, for the whole model."""
    d, w = config.head_dim, config.hidden
    names = {"model.embed_tokens.weight": (config.vocab, w), "model.norm.weight": (w,)}
    if not tied:
        names["lm_head.weight"] = (config.vocab, w)
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        names.update({
            prefix + "self_attn.q_proj.weight": (config.heads * d, w),
            prefix + "self_attn.k_proj.weight": (config.kv_heads * d, w),
            prefix + "self_attn.v_proj.weight": (config.kv_heads * d, w),
            prefix + "self_attn.o_proj.weight": (w, config.heads * d),
            prefix + "mlp.gate_proj.weight": (config.ffn, w),
            prefix + "mlp.up_proj.weight": (config.ffn, w),
            prefix + "mlp.down_proj.weight": (w, config.ffn),
            prefix + "input_layernorm.weight": (w,),
            prefix + "post_attention_layernorm.weight": (w,),
        })
    return names


def _ignored(name: str) -> bool:
    return name.endswith("rotary_emb.inv_freq")   # a buffer older exports carry; the decoder builds its own table


def check_keys(snapshot: Snapshot, expected: dict) -> None:
    """Names the checkpoint lacks and names the model does not have are both errors (checkpoint.rs:140-190), and so
    is a tensor of the wrong shape."""
    have = {name for name in snapshot.names() if not _ignored(name)}
    missing, unexpected = sorted(set(expected) - have), sorted(have - set(expected))
    if missing or unexpected:
        raise CheckpointError(f"checkpoint keys: missing {missing[:8]}{'...' if len(missing) > 8 else ''}, "
                              f"unexpected {unexpected[:8]}{'...' if len(unexpected) > 8 else ''}")
    for name, shape in expected.items():
        found = tuple(snapshot.array(name).shape)
        if found != tuple(shape):
            raise CheckpointError(f"{name}: shape {found}, expected {tuple(shape)}")


def _to_device(array: np.ndarray, kind: str):
    """A (slice of a) checkpoint array as a contiguous bf16 tensor on the current CUDA device (``convert: true`` of the
    reference's CheckpointOptions: other float types are cast)."""
    import torch

    host = np.array(array, copy=True)   # out of the read-only memory map, contiguous
    if kind == "BF16":
        return torch.from_numpy(host.view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(host).cuda().to(torch.bfloat16)


def load_llama(directory: str, shard: Shard | None = None, shard_lm_head: bool = True, interleave_gate_up: bool = True):
    """Reads a snapshot and returns ``(config, weights)`` where ``weights`` is what ``LlamaDecoder(weights=...)`` takes,
    already cut for ``shard`` (layer entries carry the fused ``wqkv`` / ``w_gate_up`` shards, so the decoder does
    not cut them again).  ``interleave_gate_up`` must equal the decoder's ``fuse_swiglu``."""
    import torch

    shard = shard or Shard()
    config = read_config(directory)
    tied = tied_embeddings(directory)
    snapshot = Snapshot(directory)
    check_keys(snapshot, llama_names(config, tied))
    tp = shard.world
    if config.heads % tp or config.kv_heads % tp or config.ffn % tp:
        raise CheckpointError("heads, kv_heads and ffn must divide by the tensor-parallel size")
    d = config.head_dim
    hs, gs, fs = shard.slice(config.heads), shard.slice(config.kv_heads), shard.slice(config.ffn)
    rows = lambda s: slice(s.start * d, s.stop * d)

    def take(name, row_slice=None, column_slice=None):
        array = snapshot.array(name)
        if row_slice is not None:
            array = array[row_slice]
        if column_slice is not None:
            array = array[:, column_slice]
        return _to_device(array, snapshot.dtype(name))

    layers = []
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        gate = take(prefix + "mlp.gate_proj.weight", fs)
        up = take(prefix + "mlp.up_proj.weight", fs)
        gate_up = (torch.stack([gate, up], 1).reshape(2 * gate.shape[0], gate.shape[1]) if interleave_gate_up
                   else torch.cat([gate, up]))
        layers.append({
            "wqkv": torch.cat([take(prefix + "self_attn.q_proj.weight", rows(hs)),
                               take(prefix + "self_attn.k_proj.weight", rows(gs)),
                               take(prefix + "self_attn.v_proj.weight", rows(gs))]).contiguous(),
            "wo": take(prefix + "self_attn.o_proj.weight", None, rows(hs)).contiguous(),
            "w_gate_up": gate_up.contiguous(),
            "w_down": take(prefix + "mlp.down_proj.weight", None, fs).contiguous(),
            "attn_norm": take(prefix + "input_layernorm.weight"),
            "mlp_norm": take(prefix + "post_attention_layernorm.weight"),
        })
    head_name = "model.embed_tokens.weight" if tied else "lm_head.weight"
    cut_head = shard_lm_head and tp > 1
    weights = {
        "layers": layers,
        "embed": take("model.embed_tokens.weight"),
        "final_norm": take("model.norm.weight"),
        "lm_head": take(head_name, shard.slice(config.vocab) if cut_head else None),
        "lm_head_is_cut": cut_head,
        "gate_up_interleaved": interleave_gate_up,
    }
    return config, weights
