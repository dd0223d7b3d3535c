"""The generation loop's decisions, kept apart from the device so they can be tested anywhere: which requests form a
batch, which sequences are still running after each step, why each one ended.

Rules per sequence (reference: src/etalii_dllm/generation.py:277-330): while fewer than max_tokens were produced and
the context is shorter than the window, run the model and choose a token; a stop token ends the sequence with
"stop" and is not part of the output; otherwise the token is appended. Running out of max_tokens or window ends it
with "length". A prompt that fills the window is refused (generation.py:519-523)."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Sequence

import numpy as np


class ContextLengthError(ValueError):
    """The prompt does not fit the context window."""


@dataclass(frozen=True)
class GenerationResult:
    tokens: tuple[int, ...]
    prompt_tokens: int
    finish_reason: str
    """"stop" (a stop token was chosen) or "length" (max_tokens or the context window)."""

    @property
    def fingerprint(self) -> str:
        """SHA-256 of the generated ids as little-endian int32 (src/etalii_dllm/generation.py:86-89)."""
        return hashlib.sha256(np.asarray(self.tokens, dtype="<i4").tobytes()).hexdigest()


def check_prompts(prompts: Sequence[Sequence[int]], vocab_size: int, context_length: int) -> None:
    """Raises for an empty prompt, a prompt that fills the context window, or a token outside the vocabulary (one
    vectorised look at each prompt: lists of thousands of ids are common)."""
    for index, prompt in enumerate(prompts):
        if len(prompt) == 0:
            raise ValueError(f"prompt {index} is empty")
        if len(prompt) >= context_length:
            raise ContextLengthError(
                f"the prompt has {len(prompt)} tokens; the context window holds {context_length}")
        tokens = np.asarray(prompt)
        outside = (tokens < 0) | (tokens >= vocab_size)
        if outside.any():
            token = tokens[int(np.argmax(outside))]
            raise ValueError(f"prompt {index}: token {token} is outside the vocabulary of {vocab_size}")


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, context_length: int, page_size: int,
                 total_pages: int, total_slots: int, max_batch: int | None = None) -> list[list[int]]:
    """Splits requests, in order, into batches that fit the cache: a sequence may grow to
    min(prompt + max_new_tokens, context_length) tokens and holds whole pages; a batch holds at most `total_slots`
    (or `max_batch`) sequences. Raises if one request alone does not fit."""
    batches: list[list[int]] = []
    current: list[int] = []
    pages = 0
    limit = min(total_slots, max_batch) if max_batch else total_slots
    for index, length in enumerate(prompt_lengths):
        need = -(-min(length + max_new_tokens, context_length) // page_size)
        if need > total_pages:
            raise ContextLengthError(
                f"request {index} needs {need * page_size} cached tokens; the cache holds {total_pages * page_size}")
        if current and (pages + need > total_pages or len(current) >= limit):
            batches.append(current)
            current, pages = [], 0
        current.append(index)
        pages += need
    if current:
        batches.append(current)
    return batches


@dataclass
class BatchRun:
    """One batch of sequences that start together. `active` lists the positions (within the batch) still running;
    `accept` takes the tokens chosen for them in that order and says which ended."""

    prompt_lengths: list[int]
    max_new_tokens: int
    stop_ids: frozenset
    context_length: int
    outputs: list[list[int]] = field(default_factory=list)
    finish: list[str | None] = field(default_factory=list)
    active: list[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        n = len(self.prompt_lengths)
        self.outputs = [[] for _ in range(n)]
        self.finish = [None] * n
        # a sequence that may produce nothing never runs (max_tokens 0: no token, reason "length")
        self.active = [i for i in range(n) if self.max_new_tokens > 0]
        for i in range(n):
            if self.max_new_tokens <= 0:
                self.finish[i] = "length"

    def accept(self, tokens: Sequence[int]) -> list[int]:
        """Applies the chosen tokens to the active sequences; returns the batch positions that ended now."""
        assert len(tokens) == len(self.active)
        ended, still = [], []
        for position, token in zip(self.active, tokens):
            token = int(token)
            if token in self.stop_ids:
                self.finish[position] = "stop"
                ended.append(position)
                continue
            self.outputs[position].append(token)
            produced = len(self.outputs[position])
            if produced >= self.max_new_tokens or self.prompt_lengths[position] + produced >= self.context_length:
                self.finish[position] = "length"
                ended.append(position)
            else:
                still.append(position)
        self.active = still
        return ended

    def steps_left(self) -> int:
        """How many more tokens every active sequence may still produce before a length limit ends one."""
        return min(min(self.max_new_tokens - len(self.outputs[p]),
                       self.context_length - self.prompt_lengths[p] - len(self.outputs[p]))
                   for p in self.active)

    def results(self) -> list[GenerationResult]:
        return [GenerationResult(tuple(out), n, reason or "length")
                for out, n, reason in zip(self.outputs, self.prompt_lengths, self.finish)]


def run_batches(prompts: Sequence[Sequence[int]], batches: Sequence[Sequence[int]],
                make_run: Callable[[list[int]], BatchRun], start: Callable, prefill: Callable, decode: Callable,
                finish: Callable, chunk: int = 16, free_chunk: int | None = None) -> list[GenerationResult]:
    """Drives batches one after another. `start(indices) -> handle` takes cache room for a batch;
    `prefill(handle, positions, prompts) -> tokens` runs the whole prompts of the named batch positions and chooses
    each one's first token; `decode(handle, positions, last_tokens, steps) -> [step][position] tokens` runs up to
    `steps` single-token steps without looking at the tokens in between; `finish(handle, positions)` gives back
    what ended sequences hold (None: everything, after an error).

    A sequence that ends inside a run of decode steps keeps its place until the run is over; what was chosen for
    it after its end is dropped. A batch without stop tokens can only end by length, which is known beforehand:
    there the host has nothing to decide in between and a run may take `free_chunk` steps (if given) at a time."""
    results: list[GenerationResult | None] = [None] * len(prompts)
    for indices in batches:
        run = make_run(list(indices))
        handle = start(list(indices))
        try:
            idle = [p for p in range(len(indices)) if p not in run.active]
            if idle:
                finish(handle, idle)
            last: dict[int, int] = {}
            first = True
            while run.active:
                positions = list(run.active)
                if first:
                    steps = [prefill(handle, positions, [prompts[indices[p]] for p in positions])]
                    first = False
                else:
                    at_most = free_chunk if free_chunk and not run.stop_ids else chunk
                    steps = decode(handle, positions, [last[p] for p in positions], min(at_most, run.steps_left()))
                ended: list[int] = []
                for chosen in steps:
                    by_position = dict(zip(positions, chosen))
                    live = list(run.active)
                    if not live:
                        break
                    ended += run.accept([by_position[p] for p in live])
                    for p in live:
                        last[p] = int(by_position[p])
                if ended:
                    finish(handle, ended)
        except BaseException:
            finish(handle, None)
            raise
        for position, result in zip(indices, run.results()):
            results[position] = result
    return results  # type: ignore[return-value]
