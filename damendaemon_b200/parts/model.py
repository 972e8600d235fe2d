"""A decoder assembled from parts according to a ModelSpec. Architecture-agnostic."""
from __future__ import annotations

from . import attention, block, embedding, feed_forward, head, norms, positions  # noqa: F401  (register the built-in parts)
from .registry import ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, lookup


def tensor_decls(spec):
    """Every checkpoint tensor the model wants, each name once."""
    decls = list(lookup(EMBEDDINGS, spec.embedding, "embedding").tensor_decls(spec.embedding))
    decls += lookup(POSITIONS, spec.position, "position encoding").tensor_decls(spec.position)
    for layer in spec.layers:
        for norm in layer.norms:
            decls += lookup(NORMS, norm, "norm").tensor_decls(norm)
        decls += lookup(MIXERS, layer.mixer, "mixer").tensor_decls(layer.mixer)
        decls += lookup(FEED_FORWARDS, layer.feed_forward, "feed-forward").tensor_decls(layer.feed_forward)
    decls += lookup(HEADS, spec.head, "head").tensor_decls(spec.head)
    unique = {}
    for d in decls:
        if d.name in unique and unique[d.name] != d:
            raise ValueError(f"tensor {d.name} is declared twice with different shapes or roles")
        unique[d.name] = d
    return list(unique.values())


def cache_needs(spec):
    """One list of cache needs per stop of the run order (empty for a stop that reads another's cache)."""
    needs = []
    for entry in spec.run_order:
        mixer = spec.layers[entry.layer].mixer
        needs.append([] if entry.cache_of is not None else list(lookup(MIXERS, mixer, "mixer").cache_needs(mixer)))
    return needs


class DecoderModel:
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        for stop, entry in enumerate(spec.run_order):
            if not 0 <= entry.layer < len(spec.layers):
                raise ValueError(f"stop {stop} of the run order names layer {entry.layer}; the model has {len(spec.layers)}")
            if entry.cache_of is not None and (not 0 <= entry.cache_of < stop or
                                               spec.run_order[entry.cache_of].cache_of is not None):
                raise ValueError(f"stop {stop} reads the cache of stop {entry.cache_of}, which must be an earlier stop "
                                 "with a cache of its own")
        self.embedding = lookup(EMBEDDINGS, spec.embedding, "embedding")(spec.embedding, weights, runtime)
        self.position = lookup(POSITIONS, spec.position, "position encoding")(spec.position, weights, runtime)
        self.blocks, self.mixers, self.feed_forwards = [], [], []
        for layer in spec.layers:
            mixer = lookup(MIXERS, layer.mixer, "mixer")(layer.mixer, weights, runtime)
            feed = lookup(FEED_FORWARDS, layer.feed_forward, "feed-forward")(layer.feed_forward, weights, runtime)
            built_norms = [lookup(NORMS, norm, "norm")(norm, weights, runtime) for norm in layer.norms]
            self.blocks.append(lookup(ARRANGEMENTS, layer, "block arrangement")(layer, built_norms, mixer, feed))
            self.mixers.append(mixer)
            self.feed_forwards.append(feed)
        self.head = lookup(HEADS, spec.head, "head")(spec.head, weights, runtime)
        self.graph_safe = all(getattr(m, "graph_safe", False) for m in self.mixers) and \
            all(getattr(f, "graph_safe", False) for f in self.feed_forwards)
        # where the mixers like a prompt to be cut (a key block of a prompt attention kernel); 1: anywhere
        self.portion_multiple = max([int(getattr(m, "portion_multiple", 1)) for m in self.mixers] + [1])

    def forward(self, ctx, caches):
        """Run the step's tokens; float32 logits [wanted rows, vocab] (or None if none are wanted).

        caches: per stop of the run order, the LayerCache view its mixer reads (and writes, if it is its own).
        """
        x = self.embedding.forward(ctx, self.position)
        for stop, entry in enumerate(self.spec.run_order):
            x = self.blocks[entry.layer].forward(x, ctx, caches[stop], self.position)
        if ctx.n_wanted == 0:
            return None
        return self.head.forward(x, ctx)
