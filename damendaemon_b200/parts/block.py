"""Block arrangements: how a layer's norm, mixer and feed-forward are wired.

'pre_norm': x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x))  (damendaemon/gpt2.py:47-64).
"""
from __future__ import annotations

from .registry import register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    def __init__(self, spec, norm1, mixer, norm2, feed_forward):
        self.spec, self.norm1, self.mixer, self.norm2, self.feed_forward = spec, norm1, mixer, norm2, feed_forward

    def forward(self, x, ctx, cache, position):
        x = self.mixer.forward(self.norm1.forward(x), x, ctx, cache, position)
        return self.feed_forward.forward(self.norm2.forward(x), x, ctx)
