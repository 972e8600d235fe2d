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
    """One list of cache needs per layer."""
    return [list(lookup(MIXERS, layer.mixer, "mixer").cache_needs(layer.mixer)) for layer in spec.layers]


class DecoderModel:
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        for entry in spec.run_order:
            if not 0 <= entry.layer < len(spec.layers) or not 0 <= entry.cache_layer < len(spec.layers):
                raise ValueError(f"run order names layer {entry.layer} (cache of {entry.cache_layer}); "
                                 f"the model has {len(spec.layers)}")
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

    def forward(self, ctx, caches):
        """Run the step's tokens; float32 logits [wanted rows, vocab] (or None if none are wanted).

        caches: per layer, the LayerCache view the layer's mixer reads and writes.
        """
        x = kernels.embed(ctx.token_ids, ctx.positions, self.token_table, self.position.embedding_table())
        x = self.position.on_embedding(x, ctx)
        for entry in self.spec.run_order:
            x = self.blocks[entry.layer].forward(x, ctx, caches[entry.cache_layer], self.position)
        if ctx.n_wanted == 0:
            return None
        y = self.final_norm.forward(x, row_index=ctx.want_rows)
        return linear(self.runtime, y, self.head, out_dtype=torch.float32)
