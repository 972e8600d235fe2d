"""Registries from a part spec's ``kind`` to the class that implements it.

Adding a mixer, feed-forward, norm, position encoding, block arrangement, embedding or head is one
``register_*`` call with a class that has the interface in ``parts/interfaces.py``;
nothing else in the framework changes.
"""
from __future__ import annotations

MIXERS: dict = {}
FEED_FORWARDS: dict = {}
NORMS: dict = {}
POSITIONS: dict = {}
ARRANGEMENTS: dict = {}
EMBEDDINGS: dict = {}
HEADS: dict = {}


def _register(table, what):
    def register(kind, cls=None, *, replace=False):
        def put(cls):
            if kind in table and not replace and table[kind] is not cls:
                raise ValueError(f"{what} kind {kind!r} is already registered")
            table[kind] = cls
            return cls
        return put if cls is None else put(cls)
    return register


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_arrangement = _register(ARRANGEMENTS, "block arrangement")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def lookup(table, spec, what):
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise KeyError(f"no {what} registered for kind {kind!r}; known: {sorted(table)}")
    return table[kind]
