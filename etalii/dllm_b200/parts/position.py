"""Rotary position encoding: frequencies from the base and the scaling rule in float64, the table of cosines and
sines per position in float64 rounded once to float32 (reference: src/etalii_dllm/numerics.py:267-311 for the
frequencies, cpp/include/dllm/nn.hpp:501-530 for the rotation of pairs (i, i + rotary_dim/2))."""
from __future__ import annotations

import math
from typing import Mapping

import torch

from .registry import register_part


def rotary_frequencies(rotary_dim: int, theta: float, scaling: Mapping | None) -> list[float]:
    log_theta = math.log(float(theta))
    freqs = [math.exp(-(2 * i / rotary_dim) * log_theta) for i in range(rotary_dim // 2)]
    kind = "default" if not scaling else str(scaling.get("rope_type", "default"))
    if kind == "linear":
        freqs = [f / float(scaling["factor"]) for f in freqs]
    elif kind == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling.get("low_freq_factor", 1.0))
        high = float(scaling.get("high_freq_factor", 4.0))
        original = float(scaling.get("original_max_position_embeddings", 8192))
        out = []
        for f in freqs:
            wavelength = 2 * math.pi / f
            if wavelength < original / high:
                out.append(f)
            elif wavelength > original / low:
                out.append(f / factor)
            else:
                smooth = (original / wavelength - low) / (high - low)
                out.append((1 - smooth) * f / factor + smooth * f)
        freqs = out
    elif kind != "default":
        raise ValueError(f"rotary scaling {kind!r} is not supported")
    return freqs


class RotaryEmbedding:
    """Gives the mixer a table [positions, rotary_dim / 2, (cos, sin)] in float32 and the number of rotated
    dimensions. Another position encoding of this role provides the same two things (or `table() is None` for no
    rotation)."""

    def __init__(self, head_dim: int, theta: float, scaling: Mapping | None = None,
                 rotary_dim: int | None = None) -> None:
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim) if rotary_dim else self.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self._table = None

    @staticmethod
    def parameters(**_) -> dict:
        return {}

    def bind(self, tensors, rt) -> None:
        key = ("rotary", self.rotary_dim, self.theta, tuple(sorted((self.scaling or {}).items())), rt.max_length)

        def make() -> torch.Tensor:
            freqs = torch.tensor(rotary_frequencies(self.rotary_dim, self.theta, self.scaling), dtype=torch.float64)
            angles = torch.arange(rt.max_length, dtype=torch.float64)[:, None] * freqs[None, :]
            table = torch.stack([torch.cos(angles), torch.sin(angles)], dim=-1).to(torch.float32)
            return table.contiguous().to(rt.device)

        self._table = rt.shared(key, make)

    def table(self) -> torch.Tensor | None:
        return self._table


register_part("position", "rotary", RotaryEmbedding)
