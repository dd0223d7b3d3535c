"""Shared helpers of the GPU tests."""
from __future__ import annotations

import numpy as np
import torch

import plain_llama as P

TOL = {"float32": 5e-5, "bfloat16": 3e-2}
"""Largest |engine logit - plain logit| allowed, as a fraction of the largest |plain logit| of the compared rows.
float32: the reference's own bound against float64 is 2e-5 (tests/test_transformer.py:158) with float64
accumulators; ours accumulates in float32. bfloat16: activations are rounded to 8 bits of mantissa between kernels."""

CASES = {"a": (P.TINY_A, 0), "b": (P.TINY_B, 1)}


def rel_error(got, ref) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def host(tensor) -> np.ndarray:
    """A host copy (the engine's outputs are work buffers that the next step overwrites)."""
    return np.array(tensor.detach().float().cpu().numpy(), copy=True)


def model_case(tag: str, std: float = 0.08):
    config, seed = CASES[tag]
    weights = P.random_weights(config, seed, std=std)
    return dict(config), weights


def make_engine(config: dict, weights: dict, dtype: str, max_tokens: int = 2048, **kwargs):
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine

    tensors = {k: torch.from_numpy(v) for k, v in weights.items()}
    return Engine(config_from_dict(config), tensors, dtype=dtype, device="cuda:0", max_tokens=max_tokens, **kwargs)


def prompts_for(config: dict, lengths, seed: int = 11):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, config["vocab_size"], n).tolist() for n in lengths]


class PlainLogits:
    """Plain-implementation logits of whole sequences, cached per token list."""

    def __init__(self, config, weights):
        self.config, self.weights, self._memo = config, weights, {}

    def __call__(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = P.forward(self.config, self.weights, list(tokens))
        return self._memo[key]
