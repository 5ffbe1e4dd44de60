"""Shared fixtures of the decode-step tests: small Llama-shaped configs, seeded weights and cache contents."""
import numpy as np

from singe_b200 import workloads
from singe_b200.llama import LlamaConfig

TINY = LlamaConfig(layers=2, hidden=64, heads=4, kv_heads=2, head_dim=16, ffn=128, vocab=97, page_size=4)
# head_dim 128 and 16-token pages: the tiled decode kernel and the tensor-core GEMM are on this path
MEDIUM = LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=512, page_size=16)
# eight KV heads: shards across 2, 4 or 8 ranks
WIDE = LlamaConfig(layers=2, hidden=512, heads=16, kv_heads=8, head_dim=128, ffn=1024, vocab=512, page_size=16)


def make_weights(config: LlamaConfig, seed: int = 4) -> dict:
    """Full (unsharded) weights ~ N(0, 0.02) rounded to bf16, as float32 numpy arrays; norm weights near 1."""
    rng = np.random.default_rng(seed)
    d, w = config.head_dim, config.hidden
    normal = lambda *shape: workloads.normal_bf16(rng, shape, std=0.02)

    def norm():
        values = (np.float32(1.0) + np.float32(0.05) * rng.standard_normal(w, dtype=np.float32)).astype(np.float32)
        bits = values.view(np.uint32).astype(np.uint64)
        rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
        return rounded.astype(np.uint32).view(np.float32)

    layers = []
    for _ in range(config.layers):
        layers.append({"wq": normal(config.heads * d, w), "wk": normal(config.kv_heads * d, w),
                       "wv": normal(config.kv_heads * d, w), "wo": normal(w, config.heads * d),
                       "gate": normal(config.ffn, w), "up": normal(config.ffn, w), "down": normal(w, config.ffn),
                       "attn_norm": norm(), "mlp_norm": norm()})
    return {"layers": layers, "embed": workloads.normal_bf16(rng, (config.vocab, w), std=1.0),
            "lm_head": normal(config.vocab, w), "final_norm": norm()}


def make_context(config: LlamaConfig, pages: int, seed: int = 5):
    rng = np.random.default_rng(seed)
    shape = (pages, config.page_size, config.kv_heads, config.head_dim)
    keys = [workloads.normal_bf16(rng, shape) for _ in range(config.layers)]
    values = [workloads.normal_bf16(rng, shape) for _ in range(config.layers)]
    return keys, values
