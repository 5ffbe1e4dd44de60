"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

These stand in for any external dataset: every tensor is drawn from a seeded generator
(N(0,1) activations and caches, N(0,0.02) weights, uniform context lengths), nothing is read from disk.
Index structures (lengths, block tables, slot maps) are built on the host with numpy so that the CPU
oracle and the device see the same integers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class PagedDecodeCase:
    """Config 2: paged-attention decode.  Arrays are host numpy; K/V/Q are float32 values already rounded to
    the cache dtype when ``bf16`` is set."""
    batch: int
    heads: int
    kv_heads: int
    head_dim: int
    block_size: int
    physical_blocks: int
    block_table_batch_stride: int
    scale: float
    lens: np.ndarray          # int32 [batch]
    block_table: np.ndarray   # uint32 [batch, stride]

    @property
    def total_tokens(self) -> int:
        return int(self.lens.sum())

    def algorithmic_bytes(self, element_bytes: int = 2) -> int:
        """HBM bytes one decode call must move: K and V rows of every cached token once, Q in, O out, the block
        table entries and the lengths."""
        kv = self.total_tokens * 2 * self.kv_heads * self.head_dim * element_bytes
        qo = 2 * self.batch * self.heads * self.head_dim * element_bytes
        blocks = int(np.sum((self.lens.astype(np.int64) + self.block_size - 1) // self.block_size))
        return kv + qo + blocks * 4 + self.batch * 4


def paged_decode_case(seed: int = 1, batch: int = 32, heads: int = 32, kv_heads: int = 8, head_dim: int = 128,
                      block_size: int = 16, min_len: int = 128, max_len: int = 4096, spare: float = 0.10,
                      lens=None) -> PagedDecodeCase:
    rng = np.random.default_rng(seed)
    if lens is None:
        lens = rng.integers(min_len, max_len + 1, size=batch)
    lens = np.asarray(lens, dtype=np.int32)
    batch = int(lens.size)
    blocks = (lens.astype(np.int64) + block_size - 1) // block_size
    needed = int(blocks.sum())
    pool = max(1, int(math.ceil(needed * (1.0 + spare))))
    stride = max(1, int((max(int(lens.max()), max_len) + block_size - 1) // block_size))
    perm = rng.permutation(pool).astype(np.uint32)
    table = np.zeros((batch, stride), dtype=np.uint32)
    at = 0
    for b in range(batch):
        table[b, : blocks[b]] = perm[at: at + blocks[b]]
        at += int(blocks[b])
    return PagedDecodeCase(batch, heads, kv_heads, head_dim, block_size, pool, stride, 1.0 / math.sqrt(head_dim),
                           lens, table)


@dataclass
class PrefillCase:
    """Config 4: packed variable-length causal prefill with a slot-mapped KV-cache write."""
    lens: np.ndarray         # int32 [batch]
    offsets: np.ndarray      # int32 [batch]  (cu_seqlens without the last entry)
    heads: int
    kv_heads: int
    head_dim: int
    page_size: int
    pages: int
    write_pages: np.ndarray  # int64 [total]
    write_slots: np.ndarray  # int64 [total]
    block_table: np.ndarray  # uint32 [batch, stride]
    scale: float

    @property
    def total_tokens(self) -> int:
        return int(self.lens.sum())

    def causal_flops(self) -> float:
        """4 * D * H * sum L(L+1)/2: QK^T and PV over the lower triangle only."""
        tri = sum(int(l) * (int(l) + 1) // 2 for l in self.lens)
        return 4.0 * self.head_dim * self.heads * tri


def prefill_case(seed: int = 3, lens=(8192, 4096, 2048, 1024), heads: int = 32, kv_heads: int = 8,
                 head_dim: int = 128, page_size: int = 16, spare: float = 0.10) -> PrefillCase:
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, dtype=np.int32)
    offsets = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    blocks = (lens.astype(np.int64) + page_size - 1) // page_size
    pool = int(math.ceil(int(blocks.sum()) * (1.0 + spare)))
    perm = rng.permutation(pool)
    stride = int(blocks.max())
    table = np.zeros((lens.size, stride), dtype=np.uint32)
    write_pages = np.zeros(int(lens.sum()), dtype=np.int64)
    write_slots = np.zeros(int(lens.sum()), dtype=np.int64)
    base = 0
    for b, n in enumerate(lens):
        mine = perm[base: base + blocks[b]]
        table[b, : blocks[b]] = mine
        idx = np.arange(int(n))
        write_pages[offsets[b]: offsets[b] + n] = mine[idx // page_size]
        write_slots[offsets[b]: offsets[b] + n] = idx % page_size
        base += int(blocks[b])
    return PrefillCase(lens, offsets, heads, kv_heads, head_dim, page_size, pool, write_pages, write_slots, table,
                       1.0 / math.sqrt(head_dim))


GEMM_SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336)]  # (N, K) of config 3
GEMM_ROWS = [1, 16, 128, 4096]


def normal_bf16(rng: np.random.Generator, shape, std: float = 1.0) -> np.ndarray:
    """N(0, std) float32 values rounded to bf16 precision (nearest even), still stored as float32."""
    values = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
    bits = values.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(shape)
