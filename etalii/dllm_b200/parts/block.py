"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream
x in float32 (reference: src/etalii_dllm/transformer.py:493-558)."""
from __future__ import annotations

from .registry import register_part


class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        h = self.mixer_norm.forward(x, rt)
        self.mixer.forward(h, x, batch, cache, rt, write_cache)
        h = self.feed_forward_norm.forward(x, rt)
        self.feed_forward.forward(h, x, batch, rt)


register_part("block", "pre_norm", PreNormBlock)
