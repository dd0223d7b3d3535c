"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream
x in float32 (reference: src/etalii_dllm/transformer.py:493-558)."""
from __future__ import annotations

from .registry import register_part


class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    @staticmethod
    def _normed(norm, consumer, x, rt):
        # a consumer that says so gets the norm still pending and may apply it inside its own kernel
        if getattr(consumer, "accepts_pending_norm", False) and hasattr(norm, "lazy"):
            return norm.lazy(x, rt)
        return norm.forward(x, rt)

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, x, rt), x, batch, cache, rt, write_cache)
        self.feed_forward.forward(self._normed(self.feed_forward_norm, self.feed_forward, x, rt), x, batch, rt)


register_part("block", "pre_norm", PreNormBlock)
