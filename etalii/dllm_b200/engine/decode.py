"""Single-token steps that follow one another on the device: model step, token choice and feedback of the chosen
token into the next step's input, captured once per batch size as a CUDA graph and replayed. The host only fills the
batch's fixed buffers before a run of steps and reads the chosen tokens after it."""
from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from ..kernels import ops
from .batch import StepBatch, StepLayout, step_values


class DecodeGraph:
    CAPACITY = 256
    """Most steps one run may take before the host reads the tokens."""

    def __init__(self, engine, batch_size: int, options, use_graph: bool = True, max_context: int | None = None,
                 min_tokens: int = 0, blocked: tuple = ()) -> None:
        """`min_tokens`, `blocked`: while the sequences have fewer than `min_tokens` tokens of output, the token ids in
        `blocked` (the stop tokens) are taken out of the choice (src/etalii_dllm/generation.py:316, 373-381)."""
        # (a weak reference: the engine owns its graphs, and an engine that is dropped should die at once, with
        # its device and pinned memory, not wait for the cycle collector)
        self.engine, self.b, self.options, self.use_graph = weakref.proxy(engine), batch_size, options, use_graph
        b = batch_size
        device = engine.rt.device
        # one token per sequence, every row wanted, no prefill tiles; behind the step's fields, the run's own two:
        # how many steps it has taken, and how many tokens of output every sequence had when it began
        self.layout = StepLayout(b, b, b, 0, extra=(("counter", "one"), ("produced", "one")))
        self.host = torch.empty(self.layout.total, dtype=torch.int32).pin_memory()
        self.meta = torch.zeros(self.layout.total, dtype=torch.int32, device=device)
        self.history = torch.zeros(self.CAPACITY * b, dtype=torch.int32, device=device)
        self.chosen = torch.zeros(b, dtype=torch.int32, device=device)
        batch = StepBatch()
        self.layout.attach(batch, self.meta)
        self.counter, self.produced = batch.counter, batch.produced
        self.min_tokens = int(min_tokens) if blocked else 0
        self.blocked = torch.tensor(sorted(blocked), dtype=torch.int32, device=device) if self.min_tokens > 0 else None
        batch.n_seqs = batch.n_tokens = batch.n_want = b
        batch.n_tiles = 0
        batch.h_new = [1] * b
        batch.max_new = 1
        batch.is_decode = True
        # the captured step serves every length up to this bound (attention launches blocks for all of it)
        batch.max_context = min(int(max_context or engine.max_length), engine.max_length)
        batch.max_position = batch.max_context - 1
        self.batch = batch
        self.graph = None
        self.generation = -1
        self.launches_per_step = 0
        self.logits = None
        """The work buffer the captured step writes its logits to, [batch, vocab] float32: after a run of steps it
        holds the last step's logits (tests compare them with a plain implementation without a second forward).
        None where the step makes the greedy choice inside the head product (engines built with
        `decode_logits=True` always compute them)."""

    def _body(self) -> None:
        # a greedy step that masks nothing needs no logits: the head product may make the choice itself
        fused = self.options.temperature == 0 and self.blocked is None and not self.engine.decode_logits
        logits = self.logits = self.engine.model.forward(self.batch, greedy_out=self.chosen if fused else None)
        if logits is not None:
            if self.blocked is not None:
                ops.mask_tokens(logits, self.blocked, self.produced, self.counter, self.min_tokens)
            self.engine.sampler.choose(logits, self.batch.slots, self.options, out=self.chosen)
        ops.decode_advance(self.batch.tokens, self.batch.tok_pos, self.batch.start, self.chosen, self.history,
                           self.counter, self.b)

    def load(self, slots, tokens, starts, produced: int = 0) -> None:
        """Fills the fixed buffers: each sequence's slot, next input token and cached length, and how many tokens of
        output the sequences have so far."""
        values = step_values(slots, [[int(t)] for t in tokens], starts, [[0]] * self.b)
        values["counter"] = np.zeros(1, np.int32)
        values["produced"] = np.asarray([produced], np.int32)
        self.layout.write(self.host.numpy(), values)
        self.batch.h_slots, self.batch.h_start = list(slots), list(starts)
        self.meta.copy_(self.host, non_blocking=True)

    def replay(self, steps: int) -> None:
        """Runs `steps` single-token steps (after `load`); the cache must already have room for them."""
        ws = self.engine.rt.ws
        if self.use_graph and (self.graph is None or self.generation != ws.generation):
            before = ops.launches
            self._body()  # once outside a capture: builds kernels, sizes work buffers
            self.launches_per_step = ops.launches - before
            steps -= 1
            torch.cuda.synchronize()
            if steps > 0:
                # No garbage collection while the stream captures: an object that dies then and owns pinned host
                # memory (an engine that is no longer used, say) makes the allocator record an event on the
                # default stream, which is not permitted during a capture and invalidates it. Dead cycles go first.
                gc.collect()
                collecting = gc.isenabled()
                gc.disable()
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        self._body()
                finally:
                    if collecting:
                        gc.enable()
                self.graph, self.generation = graph, ws.generation
        for _ in range(steps):
            if self.use_graph:
                self.graph.replay()
            else:
                before = ops.launches
                self._body()
                self.launches_per_step = ops.launches - before

    def tokens(self, steps: int) -> list[list[int]]:
        """The tokens chosen by the last `steps` steps since `load`: [step][sequence]."""
        return self.history[: steps * self.b].view(steps, self.b).tolist()
