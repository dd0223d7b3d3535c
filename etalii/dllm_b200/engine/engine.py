"""The engine: a model folder (or a configuration and a seed) in, tokens or logits out, on one CUDA device.

`Engine.from_folder` / `Engine.from_random` build the model; `step` is the one function that runs tokens through it;
`generate` is the batched generation loop above `step`; `complete` is the reference's single-prompt call
(src/etalii_dllm/engine.py:416-595 loads, 694-748 completes)."""
from __future__ import annotations

import array
import time
from typing import Sequence

import numpy as np
import torch

from .. import architectures  # noqa: F401  (registers the built-in architectures)
from ..cache.allocators import CacheError
from ..config.registry import architecture, load_config
from ..kernels import ops
from ..sampling.options import SamplingOptions
from ..sampling.sampler import Sampler
from ..weights.loader import load_weights
from ..weights.random_init import random_tensors
from .batch import BatchBuffers
from .decode import DecodeGraph
from .generate import BatchRun, GenerationResult, check_prompts, plan_batches, run_batches
from .model import Model
from .runtime import Runtime

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype {dtype!r}: use bfloat16 or float32") from None


def _token_array(tokens) -> np.ndarray:
    """Token ids as an int64 array. A list of Python ints goes through `array.array` (about half the time of
    numpy's own conversion of a list, which looks at every element's type); anything else as numpy takes it."""
    if type(tokens) is list:
        try:
            return np.frombuffer(array.array("q", tokens), dtype=np.int64)
        except (TypeError, OverflowError):
            pass
    return np.asarray(tokens, dtype=np.int64)


class Engine:
    def __init__(self, config, tensors, dtype="bfloat16", device="cuda:0", max_tokens: int | None = None,
                 max_length: int | None = None, max_slots: int | None = None, cuda_graphs: bool = True,
                 decode_chunk: int = 16, decode_logits: bool = False) -> None:
        """`max_length`: the longest sequence the cache holds (default: the model's max_position_embeddings).
        `max_tokens`: the most tokens all live sequences hold together, each rounded up to whole pages of 64
        (default: four sequences of max_length). `cuda_graphs`: replay decode steps as CUDA graphs; switched
        off by itself when a part or block of the model declares `CAPTURABLE = False` (a part made of allocating
        torch ops: a captured graph cannot hold those). `decode_chunk`: decode steps between looks at the chosen tokens.
        `decode_logits`: decode runs always compute the logits (they stay readable in the run's buffer); by default
        a greedy run lets the head product choose the token itself and stores no logits."""
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this library has no CPU path")
        self.config = config
        self.dtype = parse_dtype(dtype)
        arch = architecture(config.model_type)
        self.spec = arch.build_spec(config)
        self.context_length = int(self.spec.max_position)
        self.max_length = int(min(max_length or self.context_length, self.context_length))
        self.max_tokens = int(max_tokens or 4 * self.max_length)
        torch.cuda.set_device(torch.device(device))
        self.rt = Runtime(device, self.dtype, self.max_length)
        self.model = Model(self.spec, tensors, self.rt, self.max_tokens, max_slots=max_slots)
        self.cache = self.model.cache
        self.vocab_size = self.spec.vocab_size
        self.buffers = BatchBuffers(self.rt.device)
        self.sampler = Sampler(self.cache.n_slots, self.vocab_size, self.rt.device, self.rt.ws)
        self.steps_run = 0
        self.cuda_graphs = bool(cuda_graphs) and self.model.capturable()
        self.decode_chunk = int(decode_chunk)
        self.decode_logits = bool(decode_logits)
        self._graphs: dict = {}
        self.stats: dict = {}

    # ---- construction ----
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **kwargs) -> "Engine":
        """Loads `folder/config.json` and its safetensors; the model class is chosen by config.json's model_type."""
        config = load_config(folder)
        spec = architecture(config.model_type).build_spec(config)
        return cls(config, load_weights(folder, spec), dtype=dtype, device=device, **kwargs)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", std: float = 0.02,
                    **kwargs) -> "Engine":
        """A model of `config` with seeded random weights (stored as bfloat16, like `write_random_model`)."""
        return cls(config, random_tensors(config, seed, torch.bfloat16, std), dtype=dtype, device=device, **kwargs)

    # ---- sequences ----
    def open(self, count: int = 1) -> list[int]:
        """Takes cache slots for `count` new sequences."""
        return self.cache.acquire(count)

    def close(self, slots: Sequence[int]) -> None:
        """Gives back the slots and everything they hold."""
        self.cache.release(slots)

    # ---- the step ----
    def step(self, slots: Sequence[int], new_tokens: Sequence[Sequence[int]],
             want: Sequence[Sequence[int]] | None = None) -> torch.Tensor | None:
        """Runs the next tokens of each sequence (whole prompts or single tokens, unequal lengths) as one packed
        batch from the cache; returns float32 logits [wanted rows, vocab] on the device in the order of `slots` and
        of `want` (`want[b]` indexes sequence b's new tokens; default: each sequence's last token), or None if no
        row is wanted. The returned tensor is a work buffer: it is overwritten by the next step.

        The step is only launched when this returns. A kernel that could not finish (a bounded wait that ran out)
        reports through a status word: call `check()` after waiting for the logits (a copy to the host, a
        synchronize); `decode` and `generate` do so themselves, and the next `step` looks before it starts."""
        if len(slots) == 0:
            return None
        ops.raise_if_failed()  # whatever an earlier step reported and nobody looked at
        if len(set(slots)) != len(slots):
            raise CacheError("a sequence appears twice in one step")  # src/etalii_dllm/transformer.py:405-406
        if want is None:
            want = [[len(t) - 1] for t in new_tokens]
        new_tokens = [_token_array(tokens) for tokens in new_tokens]  # one pass over each list
        for tokens, rows in zip(new_tokens, want):
            if tokens.ndim != 1 or tokens.size == 0:
                raise ValueError("a sequence in a step needs at least one token")
            if tokens.min() < 0 or tokens.max() >= self.vocab_size:
                raise ValueError(f"a token is outside the vocabulary of {self.vocab_size}")
            if any(not 0 <= r < len(tokens) for r in rows):
                raise ValueError("a wanted position is outside the sequence's new tokens")
        starts = []
        for slot, tokens in zip(slots, new_tokens):
            self.cache.reserve(slot, len(tokens))
            starts.append(self.cache.length(slot))
        self.cache.sync_tables()
        batch = self.buffers.fill(slots, new_tokens, starts, want)
        logits = self.model.forward(batch)
        for slot, tokens in zip(slots, new_tokens):
            self.cache.advance(slot, len(tokens))
        self.steps_run += 1
        self.last_batch = batch
        return logits

    def check(self) -> None:
        """Raises `KernelError` if a kernel of a step that has finished reported that its results are invalid."""
        ops.raise_if_failed()

    def decode(self, slots: Sequence[int], tokens: Sequence[int], steps: int,
               options: SamplingOptions | None = None, min_tokens: int = 0, blocked: Sequence[int] = (),
               produced: int = 0) -> list[list[int]]:
        """Runs `steps` single-token steps for the sequences in `slots`, starting from `tokens` (each sequence's
        latest token, not yet in the cache); every step's chosen token is the next step's input, on the device.
        Returns the chosen tokens [step][sequence]. Uses one CUDA graph per batch size and sampling options.
        `blocked` token ids cannot be chosen while a sequence has fewer than `min_tokens` tokens of output, of which
        it has `produced` now."""
        if produced >= min_tokens or not blocked:
            min_tokens, blocked = 0, ()  # nothing is held back any more: the graph without the masking kernel
        graph = self._decode_graph(len(slots), options or SamplingOptions(),
                                   max(self.cache.length(s) for s in slots) + steps, int(min_tokens),
                                   tuple(sorted(set(int(t) for t in blocked))))
        self.decode_start(graph, slots, tokens, steps, produced)
        self.last_decode_graph = graph
        graph.replay(steps)
        chosen = graph.tokens(steps)  # (waits for the steps)
        ops.raise_if_failed()
        return chosen

    def decode_start(self, graph, slots, tokens, steps: int, produced: int = 0) -> None:
        """Makes cache room for `steps` more tokens of each sequence and loads the graph's fixed buffers."""
        if steps > graph.CAPACITY:
            raise ValueError(f"at most {graph.CAPACITY} steps per run")
        if max(self.cache.length(s) for s in slots) + steps > graph.batch.max_context:
            raise ValueError("the sequences outgrow the context this decode graph was captured for")
        if len(set(slots)) != len(slots):
            raise CacheError("a sequence appears twice in one step")
        starts = []
        for slot in slots:
            self.cache.reserve(slot, steps)
            starts.append(self.cache.length(slot))
        self.cache.sync_tables()
        graph.load(slots, tokens, starts, produced)
        for slot in slots:
            self.cache.advance(slot, steps)
        self.steps_run += steps

    CONTEXT_BUCKET = 1024
    """Decode graphs are captured for contexts up to a multiple of this; a batch that outgrows its bucket moves to
    the next graph (so attention does not launch blocks for the whole cache when contexts are short)."""

    def _decode_graph(self, batch_size: int, options: SamplingOptions, longest: int | None = None,
                      min_tokens: int = 0, blocked: tuple = ()):
        bound = self.max_length if longest is None else \
            min(self.max_length, -(-int(longest) // self.CONTEXT_BUCKET) * self.CONTEXT_BUCKET)
        key = (batch_size, bound, options.temperature, options.top_k, options.top_p, options.min_p, min_tokens,
               blocked)
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._graphs[key] = DecodeGraph(self, batch_size, options, use_graph=self.cuda_graphs,
                                                    max_context=bound, min_tokens=min_tokens, blocked=blocked)
        return graph

    # ---- generation ----
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64,
                 options: SamplingOptions | None = None, stop_token_ids: Sequence[int] | None = None,
                 ignore_eos: bool = False, max_batch: int | None = None, min_tokens: int = 0,
                 seeds: Sequence[int] | None = None) -> list[GenerationResult]:
        """Generates for every prompt (lists of token ids), as many batches one after another as the cache needs.
        Stop ids default to the model's end-of-sequence ids; `stop_token_ids` adds more; `ignore_eos` drops the
        model's own; until an output has `min_tokens` tokens no stop token can be chosen: they are taken out of the
        choice (src/etalii_dllm/cli.py:427-431, src/etalii_dllm/generation.py:316, 373-381, 512-513).
        Sequence i draws from the stream of options.seed + i, or of seeds[i] where `seeds` is given (the command
        line's N choices of each of several prompts: choice c of every prompt draws from seed + c)."""
        options = options or SamplingOptions()
        if min_tokens < 0:
            raise ValueError("min_tokens must be non-negative")
        if seeds is not None and len(seeds) != len(prompts):
            raise ValueError("seeds: one per prompt")
        stats = self.stats = {"prefill_s": 0.0, "prefill_tokens": 0, "decode_s": 0.0, "decode_steps": 0,
                              "decode_tokens": 0}
        prompts = [np.asarray(p, dtype=np.int64).reshape(-1) for p in prompts]  # one pass over each list
        window = min(self.context_length, self.max_length)
        check_prompts(prompts, self.vocab_size, window)
        stops = set() if ignore_eos else set(self.spec.stop_token_ids)
        stops.update(int(t) for t in (stop_token_ids or ()))
        batches = plan_batches([len(p) for p in prompts], max_new_tokens, window, self.cache.page_size,
                               self.cache.smallest_pool(), self.cache.n_slots, max_batch)

        held_back = tuple(sorted(stops)) if min_tokens > 0 else ()
        produced = [0]  # tokens of output every running sequence of the batch has (they start together)

        def make_run(indices):
            return BatchRun([len(prompts[i]) for i in indices], max_new_tokens, frozenset(stops), window)

        def start(indices):
            produced[0] = 0
            slots = self.open(len(indices))
            if options.temperature > 0:
                self.sampler.seed(slots, [options.seed + i if seeds is None else int(seeds[i]) for i in indices])
            return slots

        def prefill(slots, positions, tokens):
            began = time.perf_counter()
            logits = self.step([slots[p] for p in positions], tokens)
            if held_back:
                ops.mask_tokens(logits, torch.tensor(held_back, dtype=torch.int32, device=self.rt.device),
                                torch.zeros(1, dtype=torch.int32, device=self.rt.device), None, min_tokens)
            chosen = self.sampler.choose(logits, self.last_batch.slots, options).tolist()
            ops.raise_if_failed()
            produced[0] = 1
            stats["prefill_s"] += time.perf_counter() - began
            stats["prefill_tokens"] += sum(len(t) for t in tokens)
            return chosen

        def decode(slots, positions, last_tokens, steps):
            began = time.perf_counter()
            out = self.decode([slots[p] for p in positions], last_tokens, steps, options, min_tokens, held_back,
                              produced[0])
            produced[0] += steps
            stats["decode_s"] += time.perf_counter() - began
            stats["decode_steps"] += steps
            stats["decode_tokens"] += steps * len(positions)
            return out

        def finish(slots, positions):
            if positions is None:  # an error: give everything still held back
                self.close([s for s in slots if self.cache.slots.is_held(s)])
            else:
                self.close([slots[p] for p in positions])

        return run_batches(prompts, batches, make_run, start, prefill, decode, finish, chunk=self.decode_chunk,
                           free_chunk=DecodeGraph.CAPACITY)

    def complete(self, prompt: Sequence[int], max_tokens: int = 64,
                 options: SamplingOptions | None = None, **kwargs) -> GenerationResult:
        """One prompt, the reference's call (src/etalii_dllm/engine.py:694-695), with token ids for text."""
        return self.generate([prompt], max_tokens, options, **kwargs)[0]
