"""Arrangements of a layer's parts. A block class declares the parts it takes as `PARTS` (name -> role), is built
with them as keyword arguments, exposes them as `parts` (name -> part) and its one mixer as `mixer`, and runs them
in `forward(x, batch, cache, rt, write_cache)` on the float32 residual stream x.

"pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)) (reference: src/etalii_dllm/transformer.py:493-558)."""
from __future__ import annotations

from .registry import register_part


def normed(norm, consumer, x, rt):
    """The norm's output for `consumer`: a consumer that says so gets the norm still pending and may apply it
    inside its own kernel."""
    if getattr(consumer, "accepts_pending_norm", False) and hasattr(norm, "lazy"):
        return norm.lazy(x, rt)
    return norm.forward(x, rt)


class PreNormBlock:
    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.parts = {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": mixer_norm,
                      "feed_forward_norm": feed_forward_norm}
        # each norm feeds exactly one part here, so its weight may move into that part's first product
        for norm, consumer in ((mixer_norm, mixer), (feed_forward_norm, feed_forward)):
            if hasattr(norm, "give_weight_to"):
                norm.give_weight_to(consumer)

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        self.mixer.forward(normed(self.mixer_norm, self.mixer, x, rt), x, batch, cache, rt, write_cache)
        self.feed_forward.forward(normed(self.feed_forward_norm, self.feed_forward, x, rt), x, batch, rt)


register_part("block", "pre_norm", PreNormBlock)
