"""Block arrangements: how a layer's norms, mixer and feed-forward are wired.

'pre_norm': x = x + mixer(norm[0](x)); x = x + feed_forward(norm[1](x))  (damendaemon/gpt2.py:47-64).
"""
from __future__ import annotations

from .registry import register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    def __init__(self, spec, norms, mixer, feed_forward):
        if len(norms) != 2:
            raise ValueError(f"a pre-norm block takes two norms (before the mixer, before the feed-forward), got {len(norms)}")
        self.spec, self.norms, self.mixer, self.feed_forward = spec, list(norms), mixer, feed_forward

    def forward(self, x, ctx, cache, position):
        x = self.mixer.forward(self.norms[0].forward(x), x, ctx, cache, position)
        return self.feed_forward.forward(self.norms[1].forward(x), x, ctx)
