"""Llama-shaped decode step over the C-ABI kernels, tensor-parallel across the GPUs of one box.

Host-side mirror of the reference's decode path: ``PageTable``/``DecodeStep`` (singe/src/nn/decode/step.rs),
``RotaryTable`` (singe/src/nn/layers/positional/rotary.rs:166-219), the pre-norm block
(singe/src/nn/layers/blocks/mod.rs:56-83: ``h += o(attn(norm h))``, ``h += down(silu(gate(norm h)) * up(norm h))``),
``GroupedQueryAttention::decode`` (singe/src/nn/layers/attention/grouped.rs:92-115) and
``CausalLm::forward_embedded`` (singe/src/nn/layers/networks/causal_lm.rs:121-148).

The reference has no tensor parallelism; the sharding here is new behaviour on top of the same math: rank r holds
query heads and KV heads ``r*H/tp ...``, its slice of every KV cache, column shards of q/k/v and gate/up, row shards
of o_proj and down_proj, and one all-reduce (sum, bf16, NCCL) after o_proj and after down_proj.  Norms, residual
stream and embedding are replicated; the LM head is sharded by vocabulary with a gather of each shard's
(max, argmax) pair, or replicated (``shard_lm_head=False``).

torch supplies device buffers, streams, CUDA graphs and ``torch.distributed``; every computation is a call into
``libsinge_kernel_sys.so``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from . import kernel_sys as ks


# ------------------------------------------------------------------------------------------------
# PageTable: singe/src/nn/decode/step.rs:131-475 (pure host integer planning)
# ------------------------------------------------------------------------------------------------

class PageTableError(ValueError):
    pass


@dataclass
class DecodeStep:
    """The paging tensors of one step (singe/src/nn/decode/step.rs:13-30), as int64 numpy arrays."""
    tokens: np.ndarray
    positions: np.ndarray
    write_pages: np.ndarray
    write_slots: np.ndarray
    query_offsets: np.ndarray
    page_offsets: np.ndarray
    pages: np.ndarray
    last_page_lengths: np.ndarray
    last_rows: np.ndarray
    real_tokens: np.ndarray
    sequence_ids: np.ndarray


class PageTable:
    """Hands out cache pages to sequences in increasing order from page zero and writes each step's paging
    tensors.  After the pages sequences can hold comes one scratch page that held/idle rows and padding write."""

    def __init__(self, sequences: int, capacity: int, page_size: int, pool: int):
        self.page_size = page_size
        self.capacity = capacity
        self.pool = pool
        self.padding = 0
        self.free: list[int] = []
        self.pages: list[list[int]] = [[] for _ in range(sequences)]
        self.lengths: list[int] = [0] * sequences
        self.reset()

    @classmethod
    def create(cls, sequences: int, capacity: int, page_size: int) -> "PageTable":
        if sequences == 0 or capacity <= 0 or page_size <= 0:
            raise PageTableError("page table size")
        return cls(sequences, capacity, page_size, sequences * ((capacity - 1) // page_size + 1))

    @classmethod
    def create_shared(cls, sequences: int, capacity: int, page_size: int, cache_tokens: int) -> "PageTable":
        if sequences == 0 or capacity <= 0 or page_size <= 0 or cache_tokens <= 0:
            raise PageTableError("page table size")
        return cls(sequences, capacity, page_size, (cache_tokens - 1) // page_size + 1)

    def with_padding(self, padding: int) -> "PageTable":
        self.padding = padding
        return self

    def reset(self) -> None:
        self.free = list(range(self.pool - 1, -1, -1))
        self.pages = [[] for _ in self.pages]
        self.lengths = [0] * len(self.lengths)

    def release(self, sequence: int) -> None:
        if not 0 <= sequence < len(self.pages):
            raise PageTableError("decoder sequence")
        self.free.extend(reversed(self.pages[sequence]))
        self.pages[sequence] = []
        self.lengths[sequence] = 0

    def free_pages(self) -> int:
        return len(self.free)

    def page_count(self) -> int:
        return self.pool + 1

    @property
    def scratch_page(self) -> int:
        return self.pool

    def table_length(self) -> int:
        return self.pool + len(self.pages) + (self.padding + self.page_size - 1) // self.page_size

    @staticmethod
    def step_tokens(tokens) -> int:
        return sum(max(len(t), 1) for t in tokens)

    def step(self, tokens) -> DecodeStep:
        return self.step_padded(tokens, self.step_tokens(tokens))

    def step_padded(self, tokens, total: int) -> DecodeStep:
        sequences = len(self.pages)
        if len(tokens) != sequences or all(len(t) == 0 for t in tokens):
            raise PageTableError("decode step needs a slice for every sequence, and tokens in one")
        padding = total - self.step_tokens(tokens)
        if padding < 0:
            raise PageTableError("a decode step is padded to fewer rows than it has")
        if padding > self.padding:
            raise PageTableError("a decode step is padded past what its page table allows")
        padded = max(i for i, t in enumerate(tokens) if len(t) > 0)
        for length, t in zip(self.lengths, tokens):
            if length + len(t) > self.capacity:
                raise PageTableError("decoder cache capacity")
        fresh = 0
        for length, held, t in zip(self.lengths, self.pages, tokens):
            if len(t) > 0:
                end = length + len(t)
                fresh += max((end - 1) // self.page_size + 1 - len(held), 0)
        if fresh > len(self.free):
            raise PageTableError("decoder cache pages")

        flat, positions, write_pages, write_slots = [], [], [], []
        query_offsets, last_rows, real_tokens, sequence_ids, visible = [0], [], [], [], []
        for row, t in enumerate(tokens):
            held = self.pages[row]
            for token in t:
                position = self.lengths[row]
                page = position // self.page_size
                if page == len(held):
                    held.append(self.free.pop())
                flat.append(int(token))
                positions.append(position)
                write_pages.append(held[page])
                write_slots.append(position % self.page_size)
                self.lengths[row] += 1
            if len(t) == 0:
                flat.append(0)
                positions.append(min(self.lengths[row], self.capacity - 1))
                write_pages.append(self.pool)
                write_slots.append(0)
            last = len(flat) - 1
            keys = self.lengths[row]
            if row == padded:
                for position in range(self.lengths[row], self.lengths[row] + padding):
                    flat.append(0)
                    positions.append(min(position, self.capacity - 1))
                    write_pages.append(self.pool)
                    write_slots.append(position % self.page_size)
                keys += padding
            visible.append(keys)
            sequence_ids.extend([row] * (len(flat) - len(sequence_ids)))
            query_offsets.append(len(flat))
            last_rows.append(last)
            real_tokens.append(len(t))

        pages, page_offsets, last_page_lengths = [], [0], []
        for held, seen in zip(self.pages, visible):
            if seen == 0:
                pages.append(self.pool)
                last_page_lengths.append(1)
            else:
                used = (seen - 1) // self.page_size + 1
                kept = min(used, len(held))
                pages.extend(held[:kept])
                pages.extend([self.pool] * (used - kept))
                last_page_lengths.append((seen - 1) % self.page_size + 1)
            page_offsets.append(len(pages))
        pages.extend([0] * (self.table_length() - len(pages)))
        as_array = lambda values: np.asarray(values, dtype=np.int64)
        return DecodeStep(as_array(flat), as_array(positions), as_array(write_pages), as_array(write_slots),
                          as_array(query_offsets), as_array(page_offsets), as_array(pages),
                          as_array(last_page_lengths), as_array(last_rows), as_array(real_tokens),
                          as_array(sequence_ids))

    def place_prompts(self, lengths) -> None:
        """Advances every sequence by ``lengths[b]`` tokens without building step tensors (bulk prompt placement)."""
        for row, count in enumerate(lengths):
            if self.lengths[row] + count > self.capacity:
                raise PageTableError("decoder cache capacity")
            need = (self.lengths[row] + count - 1) // self.page_size + 1 - len(self.pages[row]) if count > 0 else 0
            if need > len(self.free):
                raise PageTableError("decoder cache pages")
            for _ in range(max(need, 0)):
                self.pages[row].append(self.free.pop())
            self.lengths[row] += count


# ------------------------------------------------------------------------------------------------
# model
# ------------------------------------------------------------------------------------------------

@dataclass
class LlamaConfig:
    """Llama-3-8B shape by default (singe-model/src/text/text_generation/llama/mod.rs:17-22 builds a GroupedDecoder
    from the same fields of a Hugging Face config)."""
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    eps: float = 1e-5
    theta: float = 500000.0
    page_size: int = 16


def choose_decode_splits(rows: int, key_bound: int, bytes_per_key: int, sms: int) -> int:
    """Split count for the flash-decode kernel on ``rows`` (sequence, KV head) rows of up to ``key_bound`` keys.

    A small cost model fitted to the kernel on B200 (64 sequences x 2048 keys, 1 / 2 / 4 / 8 KV heads, 2 - 12 splits):
    three CTAs are resident per SM and run in waves; a CTA streams at most about 18 GB/s (its shared-memory ring
    against the loaded memory latency) and all resident CTAs together about 6 TB/s; a wave costs about 2 us before
    its first page arrives; a last, partly filled wave still costs a whole CTA's time.  The fixed 512-key split is
    fine when the rows alone fill the machine several times; with few rows (tensor-parallel shards, small batches)
    the model picks the split that just fills one wave (6 instead of 10 splits at one KV head: 15.5 us against 20.6)."""
    slots = 3 * sms
    finest = max(1, (key_bound + 127) // 128)
    best, best_time = 1, float("inf")
    for splits in range(1, min(finest, 64) + 1):
        ctas = rows * splits
        chunk = key_bound / splits * bytes_per_key
        full, rest = divmod(ctas, slots)
        elapsed = full * (2e-6 + chunk / min(18e9, 6.0e12 / slots))
        if rest:
            elapsed += 2e-6 + chunk / min(18e9, 6.0e12 / rest)
        elapsed += 0.2e-6 * splits  # the combine reads one partial per split
        if elapsed < best_time:
            best, best_time = splits, elapsed
    return best


def rotary_tables(head_dim: int, theta: float, capacity: int):
    """cos/sin [capacity, head_dim/2] in f32: inv_freq = 1 / theta^(2i/D), angle = position * inv_freq, all in f32
    (singe/src/nn/layers/positional/rotary.rs:102-105,186-205)."""
    pairs = head_dim // 2
    inverse = (np.float32(1.0) / np.power(np.float32(theta), (2 * np.arange(pairs)).astype(np.float32)
                                          / np.float32(head_dim))).astype(np.float32)
    angles = (np.arange(capacity, dtype=np.float32)[:, None] * inverse[None, :]).astype(np.float32)
    return np.cos(angles).astype(np.float32), np.sin(angles).astype(np.float32)


@dataclass
class Shard:
    rank: int = 0
    world: int = 1
    group: object = None  # torch.distributed module when world > 1

    def slice(self, count: int) -> slice:
        if count % self.world != 0:
            raise ValueError(f"{count} does not split across {self.world} ranks")
        per = count // self.world
        return slice(self.rank * per, (self.rank + 1) * per)


def shard_layer_weights(full: dict, config: LlamaConfig, shard: Shard, interleave_gate_up: bool = False) -> dict:
    """Cuts one layer's full weights (wq [H*D, W], wk/wv [G*D, W], wo [W, H*D], gate/up [F, W], down [W, F]) into
    this rank's fused shards.  Works on numpy arrays and torch tensors alike.  ``interleave_gate_up`` lays the fused
    gate/up matrix out as rows (gate_0, up_0, gate_1, up_1, ...), the layout the SwiGLU-fused GEMM reads."""
    d = config.head_dim
    hs, gs, fs = shard.slice(config.heads), shard.slice(config.kv_heads), shard.slice(config.ffn)
    rows = lambda s: slice(s.start * d, s.stop * d)
    is_numpy = isinstance(full["wq"], np.ndarray)
    cat = np.concatenate if is_numpy else __import__("torch").cat
    gate, up = full["gate"][fs], full["up"][fs]
    if interleave_gate_up:
        stack = np.stack if is_numpy else __import__("torch").stack
        gate_up = stack([gate, up], 1).reshape(2 * gate.shape[0], gate.shape[1])
    else:
        gate_up = cat([gate, up])
    return {
        "wqkv": cat([full["wq"][rows(hs)], full["wk"][rows(gs)], full["wv"][rows(gs)]]),
        "wo": full["wo"][:, rows(hs)],
        "w_gate_up": gate_up,
        "w_down": full["down"][:, fs],
        "attn_norm": full["attn_norm"],
        "mlp_norm": full["mlp_norm"],
    }


# Largest tensor-parallel degree at which collective="peer" means the one-shot kernel.
PEER_ONE_SHOT_UP_TO = 4


class LlamaDecoder:
    """One rank of a tensor-parallel Llama decoder: weights, KV caches, page table and the decode step."""

    def __init__(self, config: LlamaConfig, sequences: int, capacity: int, shard: Shard | None = None, seed: int = 4,
                 weights: dict | None = None, shard_lm_head: bool = True, max_splits: int = 0,
                 collective: str = "peer", fuse_swiglu: bool = True, overlap: bool = True, warm_mb: int = 0,
                 fold_in_kernel: bool = False, fuse_attention: bool = True):
        import torch

        self.torch = torch
        self.config = config
        self.shard = shard or Shard()
        self.sequences = sequences
        self.capacity = capacity
        self.table = PageTable.create(sequences, capacity, config.page_size)
        self.shard_lm_head = shard_lm_head and self.shard.world > 1
        tp = self.shard.world
        if config.heads % tp or config.kv_heads % tp or config.ffn % tp:
            raise ValueError("heads, kv_heads and ffn must divide by the tensor-parallel size")
        self.heads = config.heads // tp
        self.kv_heads = config.kv_heads // tp
        self.ffn = config.ffn // tp
        dev = "cuda"
        bf16 = torch.bfloat16
        self.layers = []
        if weights is None:
            weights = random_weights(config, seed)
        # SwiGLU in the epilogue of the gate/up GEMM (one launch less per layer; same roundings as the separate ops)
        self.fuse_swiglu = fuse_swiglu
        # Weights are parameters and the page table is uploaded before the step's kernels are enqueued, so the
        # kernels may fetch them while the kernel before is still running (SINGE_HINT_*).
        self.weight_hints = ks.HINT_STABLE_WEIGHTS if overlap else 0
        self.paging_hints = ks.HINT_STABLE_PAGING if overlap else 0
        # L2 warm-ahead: the light kernels of a layer (norm / collective, rotary) and the attention kernel also pull
        # up to this many bytes of the weight matrix a later kernel of the layer streams into L2.
        self.warm_bytes = (warm_mb << 20) if overlap else 0
        if "gate_up_interleaved" in weights and bool(weights["gate_up_interleaved"]) != bool(fuse_swiglu):
            raise ValueError("the checkpoint's gate/up layout does not match fuse_swiglu")
        for full in weights["layers"]:
            # a layer that already carries the fused shards (singe_b200.checkpoint.load_llama) is taken as it is
            cut = full if "wqkv" in full else shard_layer_weights(full, config, self.shard,
                                                                  interleave_gate_up=fuse_swiglu)
            self.layers.append({k: self._device(v) for k, v in cut.items()})
        self.embed = self._device(weights["embed"])
        self.final_norm = self._device(weights["final_norm"])
        head = weights["lm_head"]
        if self.shard_lm_head and not weights.get("lm_head_is_cut", False):
            head = head[self.shard.slice(config.vocab)]
        self.lm_head = self._device(head)
        self.vocab_offset = self.shard.slice(config.vocab).start if self.shard_lm_head else 0
        cos, sin = rotary_tables(config.head_dim, config.theta, capacity)
        self.cos = torch.from_numpy(cos).to(dev).to(bf16)   # the table is cast to the model dtype (rotary.rs:207-212)
        self.sin = torch.from_numpy(sin).to(dev).to(bf16)
        pages = self.table.page_count()
        shape = (pages, config.page_size, self.kv_heads, config.head_dim)
        self.key_caches = [torch.zeros(shape, dtype=bf16, device=dev) for _ in range(config.layers)]
        self.value_caches = [torch.zeros(shape, dtype=bf16, device=dev) for _ in range(config.layers)]
        # persistent step buffers (device) and their pinned host mirrors
        t = sequences
        self.stride = (capacity + config.page_size - 1) // config.page_size
        i64, i32 = torch.int64, torch.int32
        self.d_tokens = torch.zeros(t, dtype=i64, device=dev)
        self.d_positions = torch.zeros(t, dtype=i64, device=dev)
        self.d_pages = torch.zeros(t, dtype=i64, device=dev)
        self.d_slots = torch.zeros(t, dtype=i64, device=dev)
        self.d_lens = torch.zeros(t, dtype=i32, device=dev)
        self.d_table = torch.zeros((t, self.stride), dtype=i32, device=dev)
        self.h_table = np.zeros((t, self.stride), dtype=np.uint32)
        self.status = torch.zeros(1, dtype=i32, device=dev)
        w = config.hidden
        self.hidden = torch.empty((t, w), dtype=bf16, device=dev)
        self.normed = torch.empty((t, w), dtype=bf16, device=dev)
        self.qkv = torch.empty((t, (self.heads + 2 * self.kv_heads) * config.head_dim), dtype=bf16, device=dev)
        self.query = torch.empty((t, self.heads, config.head_dim), dtype=bf16, device=dev)
        self.attended = torch.empty((t, self.heads * config.head_dim), dtype=bf16, device=dev)
        self.projected = torch.empty((t, w), dtype=bf16, device=dev)
        # The two collectives of a layer: "peer" = one kernel per collective that sums the ranks' partial rows out
        # of peer memory and applies the residual add + RMSNorm that follows; "nccl" = all-reduce, then the norm.
        if collective not in ("peer", "oneshot", "twophase", "pushall", "nccl"):
            raise ValueError("collective must be 'peer', 'oneshot', 'twophase', 'pushall' or 'nccl'")
        if collective == "peer":
            # one-shot: every rank pulls all partial rows; two-phase: rows are reduced by their owners and pushed
            # back.  Measured on B200 / NVSwitch at 64 rows x 4096, ms per step: one-shot is ahead with two ranks
            # (4.28 against 4.48), level with four (3.27 / 3.27) and behind with eight (2.82 against 2.45), where
            # every rank would pull 3.5 MB per collective.
            collective = "oneshot" if tp <= PEER_ONE_SHOT_UP_TO else "twophase"
        self.collective = collective
        self.peer = None
        if tp > 1 and collective == "oneshot":
            from .peer import PeerAllReduce

            self.peer = PeerAllReduce(self.shard.group, self.shard.rank, tp, t, w)
        elif tp > 1 and collective in ("twophase", "pushall"):
            from .peer import TwoPhaseAllReduce

            self.peer = TwoPhaseAllReduce(self.shard.group, self.shard.rank, tp, t, w,
                                          replicated=collective == "pushall")
        self.gate_up = torch.empty((t, 2 * self.ffn), dtype=bf16, device=dev)
        self.activated = torch.empty((t, self.ffn), dtype=bf16, device=dev)
        self.logits = torch.empty((t, self.lm_head.shape[0]), dtype=bf16, device=dev)
        self.best_value = torch.empty(t, dtype=torch.float32, device=dev)
        self.best_index = torch.empty(t, dtype=i64, device=dev)
        self.next_tokens = torch.empty(t, dtype=i64, device=dev)
        if self.shard_lm_head:
            self.all_values = torch.empty((tp, t), dtype=torch.float32, device=dev)
            self.all_indices = torch.empty((tp, t), dtype=i64, device=dev)
        # split-K scratch owned by the caller (this class), so the step allocates nothing and can be graph-captured
        fast = config.head_dim in (64, 128) and config.page_size == 16 and config.heads // config.kv_heads <= 8
        self.fast_decode = fast
        # rotary embedding, cache write and attention of a decode step in one launch (singe_decode_step_attention_bf16)
        self.fuse_attention = fuse_attention and fast
        if max_splits <= 0:
            max_splits = choose_decode_splits(sequences * self.kv_heads, self.stride * config.page_size,
                                              2 * 2 * config.head_dim,
                                              torch.cuda.get_device_properties(0).multi_processor_count)
        self.max_splits = max_splits
        self.attn_scratch = torch.empty((t, self.heads, max_splits, config.head_dim), dtype=torch.float32, device=dev)
        self.lse_scratch = torch.empty((t, self.heads, max_splits), dtype=torch.float32, device=dev)
        # Optional: with one wave of decode CTAs (three fit an SM) the last split of a row can fold the row inside the
        # decode kernel instead of a combine launch.  Measured slower on B200 (+6 us per layer at the 8-way shard's
        # shapes: the fence and the ticket sit on every CTA's exit path), so it is off unless asked for.
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        self.tickets = (torch.zeros(t * self.kv_heads, dtype=i32, device=dev)
                        if fold_in_kernel and t * self.kv_heads * max_splits <= 3 * sms else None)
        self.graph = None

    def _device(self, array):
        torch = self.torch
        if isinstance(array, np.ndarray):
            array = torch.from_numpy(np.ascontiguousarray(array))
        return array.to("cuda").to(torch.bfloat16).contiguous()

    # ---- cache / context set-up ----

    def fill_context(self, tokens_per_sequence: int, seed: int = 4) -> None:
        """Marks ``tokens_per_sequence`` tokens of every sequence as cached and fills those cache slots with N(0,1)
        values (the benchmark's stand-in for a processed prompt)."""
        torch = self.torch
        self.table.place_prompts([tokens_per_sequence] * self.sequences)
        generator = torch.Generator(device="cuda").manual_seed(seed + 1000 * self.shard.rank)
        for cache in self.key_caches + self.value_caches:
            cache.copy_(torch.randn(cache.shape, generator=generator, device="cuda").to(torch.bfloat16))
        self._refresh_block_table()

    def _refresh_block_table(self) -> None:
        for b, held in enumerate(self.table.pages):
            self.h_table[b, : len(held)] = held
        self.d_table.copy_(self.torch.from_numpy(self.h_table.view(np.int32)))

    # ---- the step ----

    def plan(self, tokens) -> DecodeStep:
        """One token per sequence -> the step's paging tensors, uploaded into the persistent device buffers."""
        torch = self.torch
        step = self.table.step([[int(t)] for t in tokens])
        self._refresh_block_table()
        self.d_tokens.copy_(torch.from_numpy(step.tokens))
        self.d_positions.copy_(torch.from_numpy(step.positions))
        self.d_pages.copy_(torch.from_numpy(step.write_pages))
        self.d_slots.copy_(torch.from_numpy(step.write_slots))
        self.d_lens.copy_(torch.from_numpy((step.positions + 1).astype(np.int32)))
        return step

    def _warm(self, weight) -> None:
        """Attaches (the first part of) a weight matrix to the next launch as an L2 warm-ahead range."""
        if self.warm_bytes > 0:
            size = min(weight.numel() * weight.element_size(), self.warm_bytes)
            self._check(ks.lib().singe_warm_l2_with_next_launch(weight.data_ptr(), size), "warm")

    def _check(self, code: int, where: str) -> None:
        if code != ks.OK:
            raise RuntimeError(f"{where}: status {code} ({ks.status_string(code)})")

    def _linear(self, out, x, weight, stream) -> None:
        m, k = x.shape
        n = weight.shape[0]
        self._check(ks.lib().singe_linear_bf16(stream, out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k,
                                               x.stride(0), weight.stride(0), out.stride(0), 0, self.weight_hints),
                    "linear")

    def _linear_raw(self, out_pointer: int, out_stride: int, x, weight, stream) -> None:
        m, k = x.shape
        n = weight.shape[0]
        self._check(ks.lib().singe_linear_bf16(stream, out_pointer, x.data_ptr(), weight.data_ptr(), m, n, k,
                                               x.stride(0), weight.stride(0), out_stride, 0, self.weight_hints),
                    "linear")

    def close(self) -> None:
        """Releases the peer-mapped buffers (collective: every rank calls it)."""
        if self.peer is not None:
            self.peer.close()
            self.peer = None

    def _all_reduce(self, tensor) -> None:
        if self.shard.world > 1:
            self.shard.group.all_reduce(tensor)

    def forward(self) -> None:
        """Enqueues one decode step on the current stream, reading the persistent step buffers."""
        torch, lib, c = self.torch, ks.lib(), self.config
        stream = int(torch.cuda.current_stream().cuda_stream)
        t, w, d = self.sequences, c.hidden, c.head_dim
        status = self.status.data_ptr()
        self._check(lib.singe_embedding_bf16(stream, self.hidden.data_ptr(), self.embed.data_ptr(),
                                             self.d_tokens.data_ptr(), 8, t, w, c.vocab, status), "embedding")
        delta = None
        for index, layer in enumerate(self.layers):
            keys, values = self.key_caches[index], self.value_caches[index]
            if self.peer is None or index == 0:
                self._warm(layer["wqkv"])
                self._check(lib.singe_add_rms_norm_bf16(stream, self.hidden.data_ptr(),
                                                        None if delta is None else delta.data_ptr(),
                                                        self.normed.data_ptr(), layer["attn_norm"].data_ptr(), t, w,
                                                        c.eps), "attn norm")
            self._linear(self.qkv, self.normed, layer["wqkv"], stream)
            self._warm(layer["wo"])
            if self.fuse_attention:
                self._check(lib.singe_decode_step_attention_bf16(
                    stream, self.attended.data_ptr(), self.attn_scratch.data_ptr(), self.lse_scratch.data_ptr(),
                    self.qkv.data_ptr(), self.qkv.stride(0), keys.data_ptr(), values.data_ptr(),
                    self.d_lens.data_ptr(), self.d_table.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                    self.d_positions.data_ptr(), self.d_pages.data_ptr(), self.d_slots.data_ptr(), 8, t, self.heads,
                    self.kv_heads, d, c.page_size, keys.shape[0], self.stride, self.max_splits, self.capacity,
                    1.0 / math.sqrt(d), self.paging_hints,
                    None if self.tickets is None else self.tickets.data_ptr(), status), "decode step attention")
            else:
                self._check(lib.singe_rotary_cache_write_bf16(
                    stream, self.query.data_ptr(), self.qkv.data_ptr(), self.qkv.stride(0), self.cos.data_ptr(),
                    self.sin.data_ptr(), self.d_positions.data_ptr(), keys.data_ptr(), values.data_ptr(),
                    self.d_pages.data_ptr(), self.d_slots.data_ptr(), 8, t, self.heads, self.kv_heads, d,
                    keys.shape[0], c.page_size, self.capacity, status), "rotary cache write")
                if self.fast_decode:
                    self._warm(layer["w_gate_up"])
                    self._check(lib.singe_paged_kv_decode_step_bf16(
                        stream, self.attended.data_ptr(), self.attn_scratch.data_ptr(), self.lse_scratch.data_ptr(),
                        self.query.data_ptr(), keys.data_ptr(), values.data_ptr(), self.d_lens.data_ptr(),
                        self.d_table.data_ptr(), t, self.heads, self.kv_heads, d, c.page_size, keys.shape[0],
                        self.stride, self.max_splits, 1.0 / math.sqrt(d), self.paging_hints,
                        None if self.tickets is None else self.tickets.data_ptr()), "decode attention")
                else:
                    self._check(lib.singe_paged_kv_decode_attention_bf16(
                        stream, self.attended.data_ptr(), self.query.data_ptr(), keys.data_ptr(), values.data_ptr(),
                        self.d_lens.data_ptr(), self.d_table.data_ptr(), t, self.heads, self.kv_heads, d, c.page_size,
                        keys.shape[0], self.stride, 1.0 / math.sqrt(d)), "decode attention")
            if self.peer is not None:
                self._linear_raw(self.peer.partial_pointer(0), w, self.attended, layer["wo"], stream)
                self._warm(layer["w_down"])
                self.peer.reduce_add_norm(stream, 0, self.hidden.data_ptr(), self.normed.data_ptr(),
                                          layer["mlp_norm"].data_ptr(), c.eps, status)
            else:
                self._linear(self.projected, self.attended, layer["wo"], stream)
                self._all_reduce(self.projected)
                self._warm(layer["w_down"])
                self._check(lib.singe_add_rms_norm_bf16(stream, self.hidden.data_ptr(), self.projected.data_ptr(),
                                                        self.normed.data_ptr(), layer["mlp_norm"].data_ptr(), t, w,
                                                        c.eps), "mlp norm")
            if self.fuse_swiglu:
                self._check(lib.singe_linear_bf16(
                    stream, self.activated.data_ptr(), self.normed.data_ptr(), layer["w_gate_up"].data_ptr(), t,
                    2 * self.ffn, w, self.normed.stride(0), layer["w_gate_up"].stride(0), self.activated.stride(0), 1,
                    self.weight_hints), "gate/up + swiglu")
            else:
                self._linear(self.gate_up, self.normed, layer["w_gate_up"], stream)
                self._check(lib.singe_silu_mul_bf16(stream, self.activated.data_ptr(), self.gate_up.data_ptr(),
                                                    self.gate_up.data_ptr() + self.ffn * 2, self.gate_up.stride(0), t,
                                                    self.ffn), "swiglu")
            if self.peer is not None:
                # the down_proj collective also applies the norm that opens the next layer (or the final norm)
                following = self.layers[index + 1]["attn_norm"] if index + 1 < len(self.layers) else self.final_norm
                self._linear_raw(self.peer.partial_pointer(1), w, self.activated, layer["w_down"], stream)
                self._warm(self.layers[index + 1]["wqkv"] if index + 1 < len(self.layers) else self.lm_head)
                self.peer.reduce_add_norm(stream, 1, self.hidden.data_ptr(), self.normed.data_ptr(),
                                          following.data_ptr(), c.eps, status)
            else:
                self._linear(self.projected, self.activated, layer["w_down"], stream)
                self._all_reduce(self.projected)
                delta = self.projected
        if self.peer is None:
            self._warm(self.lm_head)
            self._check(lib.singe_add_rms_norm_bf16(stream, self.hidden.data_ptr(), delta.data_ptr(),
                                                    self.normed.data_ptr(), self.final_norm.data_ptr(), t, w, c.eps),
                        "final norm")
        self._linear(self.logits, self.normed, self.lm_head, stream)
        self._check(lib.singe_argmax_bf16(stream, self.best_value.data_ptr(), self.best_index.data_ptr(),
                                          self.logits.data_ptr(), self.logits.stride(0), t, self.logits.shape[1],
                                          self.vocab_offset), "argmax")
        if self.shard_lm_head:
            group = self.shard.group
            group.all_gather_into_tensor(self.all_values, self.best_value)
            group.all_gather_into_tensor(self.all_indices, self.best_index)
            winner = torch.argmax(self.all_values, dim=0, keepdim=True)  # lowest rank wins ties = lowest token id
            self.next_tokens.copy_(torch.gather(self.all_indices, 0, winner).squeeze(0))
        else:
            self.next_tokens.copy_(self.best_index)

    # ---- steps of any shape: prompts, prompt chunks behind a context, idle rows ----

    def step_tokens(self, tokens):
        """Extends each sequence with its ``tokens`` (an empty list leaves a row idle) and returns the logits of each
        sequence's last token, [sequences, vocab] -- ``Decoder::step`` of the reference (singe/src/generation/mod.rs:25-36,
        ``CachedDecoder::step`` :715-744).  A step of one token per sequence takes the decode path (``step``); anything
        else is a prompt step: every new token's K/V go into the cache first, then the packed causal prefill kernel
        attends each sequence's new tokens over all of its cached keys (``causal = 2``: the queries are the sequence's
        last tokens).  A step that cannot get its pages raises before anything changed."""
        torch, lib, c = self.torch, ks.lib(), self.config
        if all(len(t) == 1 for t in tokens):
            self.step([t[0] for t in tokens])
            return self._full_logits(self.logits)
        step = self.table.step([[int(v) for v in t] for t in tokens])
        stream = int(torch.cuda.current_stream().cuda_stream)
        dev, bf16 = "cuda", torch.bfloat16
        t, s, w, d = len(step.tokens), self.sequences, c.hidden, c.head_dim
        to_device = lambda array, dtype: torch.from_numpy(np.ascontiguousarray(array)).to(dev).to(dtype)
        d_tokens, d_positions = to_device(step.tokens, torch.int64), to_device(step.positions, torch.int64)
        d_pages, d_slots = to_device(step.write_pages, torch.int64), to_device(step.write_slots, torch.int64)
        lens_q = np.diff(step.query_offsets).astype(np.int32)
        page_counts = np.diff(step.page_offsets)
        lens_kv = ((page_counts - 1) * c.page_size + step.last_page_lengths).astype(np.int32)
        stride = max(int(page_counts.max()), 1)
        table = np.zeros((s, stride), dtype=np.uint32)
        for b in range(s):
            table[b, : page_counts[b]] = step.pages[step.page_offsets[b]: step.page_offsets[b + 1]]
        d_lens_q, d_lens_kv = to_device(lens_q, torch.int32), to_device(lens_kv, torch.int32)
        d_offsets = to_device(step.query_offsets[:-1].astype(np.int32), torch.int32)
        d_table = to_device(table.view(np.int32), torch.int32)
        d_last = to_device(step.last_rows, torch.int64)
        status = self.status.data_ptr()
        hidden = torch.empty((t, w), dtype=bf16, device=dev)
        normed = torch.empty((t, w), dtype=bf16, device=dev)
        qkv = torch.empty((t, (self.heads + 2 * self.kv_heads) * d), dtype=bf16, device=dev)
        query = torch.empty((t, self.heads, d), dtype=bf16, device=dev)
        attended = torch.empty((t, self.heads * d), dtype=bf16, device=dev)
        lse = torch.empty((t, self.heads), dtype=torch.float32, device=dev)
        projected = torch.empty((t, w), dtype=bf16, device=dev)
        activated = torch.empty((t, self.ffn), dtype=bf16, device=dev)
        gate_up = None if self.fuse_swiglu else torch.empty((t, 2 * self.ffn), dtype=bf16, device=dev)
        self._check(lib.singe_embedding_bf16(stream, hidden.data_ptr(), self.embed.data_ptr(), d_tokens.data_ptr(), 8,
                                             t, w, c.vocab, status), "embedding")
        delta = None
        for index, layer in enumerate(self.layers):
            keys, values = self.key_caches[index], self.value_caches[index]
            self._check(lib.singe_add_rms_norm_bf16(stream, hidden.data_ptr(),
                                                    None if delta is None else delta.data_ptr(), normed.data_ptr(),
                                                    layer["attn_norm"].data_ptr(), t, w, c.eps), "attn norm")
            self._linear(qkv, normed, layer["wqkv"], stream)
            self._check(lib.singe_rotary_cache_write_bf16(
                stream, query.data_ptr(), qkv.data_ptr(), qkv.stride(0), self.cos.data_ptr(), self.sin.data_ptr(),
                d_positions.data_ptr(), keys.data_ptr(), values.data_ptr(), d_pages.data_ptr(), d_slots.data_ptr(), 8,
                t, self.heads, self.kv_heads, d, keys.shape[0], c.page_size, self.capacity, status),
                "rotary cache write")
            self._check(lib.singe_paged_kv_prefill_attention_bf16(
                stream, attended.data_ptr(), lse.data_ptr(), query.data_ptr(), keys.data_ptr(), values.data_ptr(),
                d_lens_q.data_ptr(), d_lens_kv.data_ptr(), d_offsets.data_ptr(), d_table.data_ptr(), s, t, self.heads,
                self.kv_heads, d, c.page_size, keys.shape[0], stride, 2, 1.0 / math.sqrt(d)), "prompt attention")
            self._linear(projected, attended, layer["wo"], stream)
            self._all_reduce(projected)
            self._check(lib.singe_add_rms_norm_bf16(stream, hidden.data_ptr(), projected.data_ptr(), normed.data_ptr(),
                                                    layer["mlp_norm"].data_ptr(), t, w, c.eps), "mlp norm")
            if self.fuse_swiglu:
                self._check(lib.singe_linear_bf16(
                    stream, activated.data_ptr(), normed.data_ptr(), layer["w_gate_up"].data_ptr(), t, 2 * self.ffn, w,
                    normed.stride(0), layer["w_gate_up"].stride(0), activated.stride(0), 1, self.weight_hints),
                    "gate/up + swiglu")
            else:
                self._linear(gate_up, normed, layer["w_gate_up"], stream)
                self._check(lib.singe_silu_mul_bf16(stream, activated.data_ptr(), gate_up.data_ptr(),
                                                    gate_up.data_ptr() + self.ffn * 2, gate_up.stride(0), t, self.ffn),
                            "swiglu")
            self._linear(projected, activated, layer["w_down"], stream)
            self._all_reduce(projected)
            delta = projected
        self._check(lib.singe_add_rms_norm_bf16(stream, hidden.data_ptr(), delta.data_ptr(), normed.data_ptr(),
                                                self.final_norm.data_ptr(), t, w, c.eps), "final norm")
        last = normed.index_select(0, d_last).contiguous()   # CausalLm::forward_embedded keeps the last rows only
        logits = torch.empty((s, self.lm_head.shape[0]), dtype=bf16, device=dev)
        self._linear(logits, last, self.lm_head, stream)
        return self._full_logits(logits)

    def _full_logits(self, logits):
        """[sequences, vocab] on every rank (the LM head may be sharded by vocabulary)."""
        if not self.shard_lm_head:
            return logits
        torch = self.torch
        pieces = [torch.empty_like(logits) for _ in range(self.shard.world)]
        self.shard.group.all_gather(pieces, logits.contiguous())
        return torch.cat(pieces, dim=1)

    def capture(self) -> None:
        """Captures ``forward`` into a CUDA graph that later steps replay (the reference replays a captured
        step the same way, singe/src/generation/mod.rs:529-579)."""
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.forward()  # warm-up outside capture: loads modules, sizes nothing (all buffers are preallocated)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.forward()

    def step(self, tokens) -> "object":
        """Plans and runs one decode step; returns the device tensor of greedy next tokens [sequences]."""
        self.plan(tokens)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.forward()
        return self.next_tokens


class CachedDecoder:
    """``LlamaDecoder`` behind the reference's ``Decoder`` trait (singe/src/generation/mod.rs:25-52), which is what
    ``singe_b200.generation`` drives: ``sequences()``, ``step(tokens)``, ``reset()``, ``release(row)``,
    ``largest_chunk()``.  Prompt steps read at most the largest prompt chunk of extra tokens (16, 64, 256, ... 1024,
    ``PromptChunks``, :367-417)."""

    def __init__(self, model: LlamaDecoder, prompt_chunks=None):
        from .generation import PromptChunks

        self.model = model
        self.chunks = (prompt_chunks or PromptChunks.STANDARD).sizes(model.capacity)

    def sequences(self) -> int:
        return self.model.sequences

    def step(self, tokens):
        return self.model.step_tokens(tokens)

    def reset(self) -> None:
        self.model.table.reset()

    def release(self, sequence: int) -> None:
        self.model.table.release(sequence)

    def largest_chunk(self):
        return self.chunks[-1] if self.chunks else 0


def random_weights(config: LlamaConfig, seed: int = 4) -> dict:
    """Random-init weights ~ N(0, 0.02) in bf16 on the GPU (norm weights 1), identical on every rank for a seed."""
    import torch

    generator = torch.Generator(device="cuda").manual_seed(seed)

    def normal(*shape):
        return (torch.randn(shape, generator=generator, device="cuda") * 0.02).to(torch.bfloat16)

    d, w = config.head_dim, config.hidden
    layers = []
    for _ in range(config.layers):
        layers.append({
            "wq": normal(config.heads * d, w), "wk": normal(config.kv_heads * d, w),
            "wv": normal(config.kv_heads * d, w), "wo": normal(w, config.heads * d),
            "gate": normal(config.ffn, w), "up": normal(config.ffn, w), "down": normal(w, config.ffn),
            "attn_norm": torch.ones(w, dtype=torch.bfloat16, device="cuda"),
            "mlp_norm": torch.ones(w, dtype=torch.bfloat16, device="cuda"),
        })
    return {"layers": layers, "embed": normal(config.vocab, w), "lm_head": normal(config.vocab, w),
            "final_norm": torch.ones(w, dtype=torch.bfloat16, device="cuda")}


def decode_step_bytes(config: LlamaConfig, sequences: int, context: int, tp: int = 1, shard_lm_head: bool = True) -> dict:
    """Algorithmic HBM bytes one rank moves per decode step: its weight shards and its slice of the KV cache."""
    d, w = config.head_dim, config.hidden
    per_layer = ((config.heads + 2 * config.kv_heads) * d * w + w * config.heads * d + 3 * config.ffn * w) // tp
    head = config.vocab * w // (tp if shard_lm_head else 1)
    weights = 2 * (config.layers * per_layer + head)
    kv_read = config.layers * sequences * context * 2 * (config.kv_heads // tp) * d * 2
    kv_write = config.layers * sequences * 2 * (config.kv_heads // tp) * d * 2
    return {"weights": weights, "kv_read": kv_read, "kv_write": kv_write, "total": weights + kv_read + kv_write}
