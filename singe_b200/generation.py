"""Generation loop over a decoder that keeps its own paged cache: continuous batching, prompt chunks, stop rules.

Host-side mirror of singe/src/generation/mod.rs (pure control flow over integer token lists; the decoder does the
computing):
  ``Decoder`` protocol            the trait at generation/mod.rs:25-52 -- ``sequences()``, ``step(tokens)`` returning the
                                  logits of each sequence's last token ``[S, V]``, ``reset()``, ``release(i)``,
                                  ``largest_chunk()``
  ``GenerationOptions``           :55-68 (greedy choice only: sampling is not part of this path)
  ``RunningBatch``                :102-232 -- sequences join free rows and leave when they finish, while the others run
  ``step_portions``               :291-307 -- how much of its pending prompt each row reads in one step
  ``generate`` / ``generate_batch``  :70-84, :309-349
  ``PromptChunks``                :367-417 -- the prompt step sizes a decoder prepares: 16, 64, 256, ... up to 1024
A step that fails (cache pages or capacity exhausted) raises before anything changed, so the caller can let a
sequence finish and try again, as the reference's ``CachedDecoder::step`` guarantees by stepping a copy of its page
table (:715-744).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


class GenerationError(ValueError):
    pass


@dataclass
class GenerationOptions:
    max_new_tokens: int = 0
    stop_tokens: list = field(default_factory=list)
    suppressed_tokens: list = field(default_factory=list)        # never chosen
    first_suppressed_tokens: list = field(default_factory=list)  # not chosen as a sequence's first token


@dataclass(frozen=True)
class GeneratedToken:
    sequence: int     # which sequence, by the order they joined
    token: int
    finished: bool    # the sequence's last token: its row is free again


@dataclass(frozen=True)
class PromptChunks:
    """The extra tokens (past one per row) of the prompt steps a decoder prepares: ``smallest``, then four times as
    many each time, up to ``largest`` and to one less than a sequence's capacity, which is always the last."""
    smallest: int = 16
    largest: int = 1024

    def sizes(self, capacity: int) -> list:
        limit = min(self.largest, max(capacity - 1, 0))
        if limit == 0:
            return []
        sizes = []
        size = max(self.smallest, 1)
        while size < limit:
            sizes.append(size)
            size *= 4
        sizes.append(limit)
        return sizes


PromptChunks.NONE = PromptChunks(0, 0)
PromptChunks.STANDARD = PromptChunks(16, 1024)


def step_portions(pending, largest):
    """How many of its ``pending`` tokens each row reads in a step: a token per running row, and up to ``largest``
    more, given to the first rows that have them.  ``largest`` None: everything."""
    if largest is None:
        return list(pending)
    spare = sum(max(tokens - 1, 0) for tokens in pending)
    extra = min(spare, largest)
    portions = []
    for tokens in pending:
        taken = min(max(tokens - 1, 0), extra)
        extra -= taken
        portions.append(min(tokens, 1) + taken)
    return portions


def _logits_array(logits) -> np.ndarray:
    if hasattr(logits, "detach"):
        logits = logits.detach().float().cpu().numpy()
    return np.asarray(logits, dtype=np.float32)


class _Running:
    def __init__(self, identifier: int, prompt):
        self.id = identifier
        self.pending = [int(t) for t in prompt]   # what its next step reads: its prompt, then the token last chosen
        self.generated = 0


class RunningBatch:
    """A batch whose sequences join and leave while the others run, each in a row of its decoder.  A finished
    sequence frees its row and its pages at once."""

    def __init__(self, decoder, options: GenerationOptions):
        if options.max_new_tokens == 0:
            raise GenerationError("a running batch generates at least one token per sequence")
        decoder.reset()
        self.decoder = decoder
        self.options = options
        self.rows = [None] * decoder.sequences()
        self.joined = 0
        self._suppression = None

    @classmethod
    def create(cls, decoder, options: GenerationOptions) -> "RunningBatch":
        return cls(decoder, options)

    def join(self, prompt):
        """Starts a sequence after ``prompt`` in a free row and returns its id, or None when every row is taken."""
        return self.join_with(prompt, lambda decoder, row: None)

    def join_with(self, prompt, prepare):
        if len(prompt) == 0:
            raise GenerationError("generation prompt is empty")
        free = [index for index, row in enumerate(self.rows) if row is None]
        if not free:
            return None
        index = free[0]
        prepare(self.decoder, index)   # a sequence whose preparation raises does not join
        identifier = self.joined
        self.rows[index] = _Running(identifier, prompt)
        self.joined += 1
        return identifier

    def is_empty(self) -> bool:
        return all(row is None for row in self.rows)

    def _suppress(self, logits: np.ndarray, first) -> np.ndarray:
        options = self.options
        if not options.suppressed_tokens and not options.first_suppressed_tokens:
            return logits
        vocabulary = logits.shape[1]
        if self._suppression is None:
            table = np.zeros((2, vocabulary), dtype=np.float32)   # row 0: later tokens, row 1: a sequence's first
            for token, rows in ([(t, (0, 1)) for t in options.suppressed_tokens]
                                + [(t, (1,)) for t in options.first_suppressed_tokens]):
                if not 0 <= token < vocabulary:
                    raise GenerationError(f"suppressed token {token} is outside a vocabulary of {vocabulary}")
                for row in rows:
                    table[row, token] = -np.inf
            self._suppression = table
        return logits + self._suppression[np.asarray(first, dtype=np.int64)]

    def advance(self):
        """Runs one step and returns the token each running sequence chose, in row order (none for a sequence still
        reading its prompt).  A step that fails changes nothing."""
        if self.is_empty():
            return []
        pending = [0 if row is None else len(row.pending) for row in self.rows]
        portions = step_portions(pending, self.decoder.largest_chunk())
        tokens = [[] if row is None else row.pending[:portion] for row, portion in zip(self.rows, portions)]
        logits = _logits_array(self.decoder.step(tokens))
        first = [row is not None and row.generated == 0 and len(row.pending) == portion
                 for row, portion in zip(self.rows, portions)]
        logits = self._suppress(logits, first)
        chosen = logits.argmax(axis=1)
        if chosen.shape[0] != len(self.rows):
            raise GenerationError("generated tokens")
        generated = []
        for index, (row, portion) in enumerate(zip(self.rows, portions)):
            if row is None:
                continue
            del row.pending[:portion]
            if row.pending:
                continue
            token = int(chosen[index])
            row.generated += 1
            finished = row.generated == self.options.max_new_tokens or token in self.options.stop_tokens
            generated.append(GeneratedToken(row.id, token, finished))
            if finished:
                self.rows[index] = None
                self.decoder.release(index)
            else:
                row.pending.append(token)
        return generated


def generate_batch(decoder, prompts, options: GenerationOptions, on_token=None):
    """Generates tokens after each of ``prompts`` (one per decoder row, lengths may differ); returns each sequence's
    tokens.  A finished sequence frees what it holds, and its row stays idle for the rest of the batch's steps."""
    if len(prompts) == 0 or any(len(prompt) == 0 for prompt in prompts):
        raise GenerationError("generation prompt is empty")
    if len(prompts) != decoder.sequences():
        raise GenerationError(f"generation prompts: expected {decoder.sequences()}, got {len(prompts)}")
    tokens = [[] for _ in prompts]
    if options.max_new_tokens == 0:
        decoder.reset()
        return tokens
    batch = RunningBatch.create(decoder, options)
    for prompt in prompts:
        batch.join(prompt)
    while not batch.is_empty():
        for generated in batch.advance():
            tokens[generated.sequence].append(generated.token)
            if on_token is not None:
                on_token(generated.sequence, generated.token)
    return tokens


def generate(decoder, prompt, options: GenerationOptions, on_token=None):
    """Generates tokens after ``prompt`` on a decoder of one sequence."""
    wrapped = None if on_token is None else (lambda _, token: on_token(token))
    return generate_batch(decoder, [prompt], options, wrapped)[0]
