"""A decoder assembled from parts according to a ModelSpec. Architecture-agnostic."""
from __future__ import annotations

import torch

from .. import kernels
from . import attention, block, feed_forward, norms, positions  # noqa: F401  (register the built-in parts)
from .linear import linear
from .registry import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, lookup
from .spec import TensorDecl


def tensor_decls(spec):
    """Every checkpoint tensor the model wants, each name once."""
    decls = [TensorDecl(spec.token_table, (spec.vocab_size, spec.width), "table")]
    decls += lookup(POSITIONS, spec.position, "position encoding").tensor_decls(spec.position)
    for layer in spec.layers:
        decls += lookup(NORMS, layer.norm1, "norm").tensor_decls(layer.norm1)
        decls += lookup(MIXERS, layer.mixer, "mixer").tensor_decls(layer.mixer)
        decls += lookup(NORMS, layer.norm2, "norm").tensor_decls(layer.norm2)
        decls += lookup(FEED_FORWARDS, layer.feed_forward, "feed-forward").tensor_decls(layer.feed_forward)
    decls += lookup(NORMS, spec.final_norm, "norm").tensor_decls(spec.final_norm)
    if spec.head_weight:
        decls.append(TensorDecl(spec.head_weight, (spec.vocab_size, spec.width), "matrix"))
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
        self.token_table = weights[spec.token_table]
        self.head = weights[spec.head_weight] if spec.head_weight else self.token_table
        self.position = lookup(POSITIONS, spec.position, "position encoding")(spec.position, weights, runtime)
        self.blocks = []
        for layer in spec.layers:
            self.blocks.append(lookup(ARRANGEMENTS, layer, "block arrangement")(
                layer,
                lookup(NORMS, layer.norm1, "norm")(layer.norm1, weights, runtime),
                lookup(MIXERS, layer.mixer, "mixer")(layer.mixer, weights, runtime),
                lookup(NORMS, layer.norm2, "norm")(layer.norm2, weights, runtime),
                lookup(FEED_FORWARDS, layer.feed_forward, "feed-forward")(layer.feed_forward, weights, runtime)))
        self.final_norm = lookup(NORMS, spec.final_norm, "norm")(spec.final_norm, weights, runtime)
        self.graph_safe = all(getattr(b.mixer, "graph_safe", False) and getattr(b.feed_forward, "graph_safe", False)
                              for b in self.blocks)

    def forward(self, ctx, caches):
        """Run the step's tokens; float32 logits [wanted rows, vocab] (or None if none are wanted).

        caches: per stop of the run order, the LayerCache view its mixer reads (and writes, if it is its own).
        """
        x = kernels.embed(ctx.token_ids, ctx.positions, self.token_table, self.position.embedding_table())
        x = self.position.on_embedding(x, ctx)
        for stop, entry in enumerate(self.spec.run_order):
            x = self.blocks[entry.layer].forward(x, ctx, caches[stop], self.position)
        if ctx.n_wanted == 0:
            return None
        y = self.final_norm.forward(x, row_index=ctx.want_rows)
        return linear(self.runtime, y, self.head, out_dtype=torch.float32)
