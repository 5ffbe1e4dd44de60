"""CPU restatement of one Llama decode step -- TEST INFRASTRUCTURE ONLY (never imported by the package).

Follows the reference's eager bf16 path op by op, rounding to bf16 where a tensor op would return a bf16 tensor
(the CPU backend widens bf16 to f32, computes, and rounds the result: singe/src/backend/kernels.rs:662-705):
  CausalLm::forward_embedded      singe/src/nn/layers/networks/causal_lm.rs:121-148
  PreNormBlock::run               singe/src/nn/layers/blocks/mod.rs:56-83
  GroupedQueryAttention::decode   singe/src/nn/layers/attention/grouped.rs:92-115
  RotaryAngles::rotate_pairs      singe/src/nn/layers/positional/rotary.rs:274-304 (table cast to bf16, :207-212)
  KvCache::write                  singe/src/nn/decode/cache.rs:97-101
  Tensor::paged_attention (CPU)   singe/src/backend/cpu/normalization/attention.rs:297-540
  GatedMlp::forward               singe/src/nn/layers/feed_forward/mod.rs:58-66
  Linear::forward                 singe/src/nn/layers/linear/mod.rs:49-70
All arrays are float32 holding bf16-representable values.
"""
from __future__ import annotations

import numpy as np

from . import oracle


def bf16(x: np.ndarray) -> np.ndarray:
    return oracle.round_to_bf16(np.ascontiguousarray(x, dtype=np.float32)).reshape(np.shape(x))


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    m, k = x.shape
    n = weight.shape[0]
    bits = oracle.linear_bf16(oracle.f32_to_bf16_bits(x), oracle.f32_to_bf16_bits(weight), m=m, n=n, k=k)
    return oracle.bf16_bits_to_f32(bits).reshape(m, n)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return bf16(oracle.rms_norm_f32(x, weight, eps))


def rotate(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x [T, H, D]; cos/sin [T, D/2] already rounded to bf16.  Each tensor op rounds: mul, mul, then sub/add."""
    half = x.shape[-1] // 2
    first, second = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    rotated_first = bf16(bf16(first * c) - bf16(second * s))
    rotated_second = bf16(bf16(second * c) + bf16(first * s))
    return np.concatenate([rotated_first, rotated_second], axis=-1)


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    activated = bf16(gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)))
    return bf16(activated * up)


def decode_step(config, weights: dict, key_caches, value_caches, step, cos_table, sin_table):
    """Runs one step for every sequence.  ``weights`` holds full (unsharded) float32 arrays per layer;
    ``key_caches``/``value_caches`` are lists of [P, S, G, D] float32 arrays, updated in place;
    ``step`` is a PageTable DecodeStep.  Returns logits [sequences, vocab] (bf16-rounded float32)."""
    tokens = step.tokens
    t = tokens.shape[0]
    d = config.head_dim
    hidden = weights["embed"][tokens]
    cos = bf16(cos_table)[step.positions]
    sin = bf16(sin_table)[step.positions]
    scale = np.float32(1.0 / np.sqrt(d))
    for index, layer in enumerate(weights["layers"]):
        normed = rms_norm(hidden, layer["attn_norm"], config.eps)
        query = rotate(linear(normed, layer["wq"]).reshape(t, config.heads, d), cos, sin)
        key = rotate(linear(normed, layer["wk"]).reshape(t, config.kv_heads, d), cos, sin)
        value = linear(normed, layer["wv"]).reshape(t, config.kv_heads, d)
        assert oracle.kv_cache_write(key_caches[index], np.ascontiguousarray(key), step.write_pages,
                                     step.write_slots) == oracle.OK
        assert oracle.kv_cache_write(value_caches[index], np.ascontiguousarray(value), step.write_pages,
                                     step.write_slots) == oracle.OK
        status, attended, _ = oracle.attend_paged_f32(
            query, key_caches[index], value_caches[index], step.query_offsets, step.page_offsets, step.pages,
            step.last_page_lengths, scale=float(scale), causal=True)
        assert status == oracle.OK
        attended = bf16(attended).reshape(t, config.heads * d)
        hidden = bf16(hidden + linear(attended, layer["wo"]))
        normed = rms_norm(hidden, layer["mlp_norm"], config.eps)
        fed = linear(silu_mul(linear(normed, layer["gate"]), linear(normed, layer["up"])), layer["down"])
        hidden = bf16(hidden + fed)
    normed = rms_norm(hidden, weights["final_norm"], config.eps)
    return linear(normed[step.last_rows], weights["lm_head"])
