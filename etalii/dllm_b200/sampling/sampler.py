"""Token choice on the device for a batch of rows of logits, one random stream per sequence kept in the sequence's
slot (xoshiro256** seeded through SplitMix64, as cpp/include/dllm/random.hpp:11-55)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .options import SamplingOptions


class Sampler:
    def __init__(self, n_slots: int, vocab_size: int, device, workspace) -> None:
        """`workspace`: the engine's work buffers. The scratch of temperature sampling is one of them, so that a
        captured decode graph, which holds the scratch's address, is dropped like any other graph when the buffer
        is replaced by a larger one (the workspace counts its reallocations and graphs compare the count)."""
        self.device, self.vocab_size = device, vocab_size
        self.rng = torch.zeros((n_slots, 4), dtype=torch.int64, device=device)
        self.ws = workspace

    def seed(self, slots: list[int], seeds: list[int]) -> None:
        """Starts the stream of each slot from its seed (modulo 2^64)."""
        wrapped = [((s % (1 << 64)) + (1 << 63)) % (1 << 64) - (1 << 63) for s in seeds]  # as signed 64-bit patterns
        rows = torch.tensor(slots, dtype=torch.int32, device=self.device)
        ops.seed_rng(self.rng, rows, torch.tensor(wrapped, dtype=torch.int64, device=self.device))

    def choose(self, logits: torch.Tensor, slots: torch.Tensor, options: SamplingOptions,
               out: torch.Tensor | None = None) -> torch.Tensor:
        """One token per row of `logits` [rows, vocab]; `slots` (int32, device) names each row's random stream."""
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=self.device)
        scratch = None
        if options.temperature > 0:
            scratch = self.ws.buffer("sample_scratch", (ops.sample_scratch(rows, logits.shape[1]),), torch.float32)
        ops.sample(out, logits, scratch, self.rng if scratch is not None else None,
                   slots if scratch is not None else None, options.temperature, options.top_k, options.top_p,
                   options.min_p)
        return out
