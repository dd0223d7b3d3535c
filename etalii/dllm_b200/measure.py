"""Timing of whole generation calls, after the reference's harness (benchmarks/benchmark.py:191-216): one warm-up
call, then several repetitions that each start from an empty cache, the wall clock around the whole call (prompt
step, decoding, token lists back on the host), and mean and standard deviation over the repetitions."""
from __future__ import annotations

import math
import time
from typing import Sequence

from .sampling.options import SamplingOptions


def mean_sd(values: Sequence[float]) -> tuple[float, float]:
    n = len(values)
    mean = sum(values) / n
    sd = math.sqrt(sum((v - mean) ** 2 for v in values) / (n - 1)) if n > 1 else 0.0
    return mean, sd


def measure_generation(engine, prompts: Sequence[Sequence[int]], new_tokens: int,
                       options: SamplingOptions | None = None, repeats: int = 5, warmup: int = 1) -> dict:
    """Calls `engine.generate(prompts, new_tokens, ignore_eos=True)` `warmup + repeats` times and returns, over the
    repetitions: generated tokens per second of the whole call (`tokens_per_s`, `sd`), the seconds of a call and of
    its prompt and decode parts, prompt tokens per second of the prompt part and decoded tokens per second of the
    decode part."""
    import torch

    options = options or SamplingOptions()
    rates, totals, prefill, decode, prefill_rate, decode_rate = [], [], [], [], [], []
    for index in range(warmup + repeats):
        torch.cuda.synchronize()
        began = time.perf_counter()
        results = engine.generate(prompts, new_tokens, options, ignore_eos=True)
        elapsed = time.perf_counter() - began
        if index < warmup:
            continue
        stats = engine.stats
        produced = sum(len(r.tokens) for r in results)
        rates.append(produced / elapsed)
        totals.append(elapsed)
        prefill.append(stats["prefill_s"])
        decode.append(stats["decode_s"])
        if stats["prefill_s"] > 0:
            prefill_rate.append(stats["prefill_tokens"] / stats["prefill_s"])
        if stats["decode_s"] > 0:
            decode_rate.append(stats["decode_tokens"] / stats["decode_s"])
    rate, sd = mean_sd(rates)
    return {
        "tokens_per_s": rate, "sd": sd, "repeats": repeats, "call_s": mean_sd(totals)[0],
        "prefill_s": mean_sd(prefill)[0], "decode_s": mean_sd(decode)[0],
        "prefill_tokens_per_s": mean_sd(prefill_rate)[0] if prefill_rate else 0.0,
        "decode_tokens_per_s": mean_sd(decode_rate)[0] if decode_rate else 0.0,
    }


def random_prompts(vocab_size: int, lengths: Sequence[int], seed: int = 0) -> list[list[int]]:
    """Seeded random token ids of the given lengths (synthetic prompts for measurements)."""
    import numpy as np

    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab_size, int(n)).tolist() for n in lengths]
