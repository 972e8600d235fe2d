"""Embeddings: from the step's token ids to the float32 residual stream.

'tokens': x[t] = table[id[t]] (+ the position encoding's own table at the token's position, if it has one:
damendaemon/gpt2.py:46), one fused gather; the position encoding may then act on x (``on_embedding``).
"""
from __future__ import annotations

from .. import kernels
from .interfaces import Embedding
from .registry import register_embedding
from .spec import TensorDecl


@register_embedding("tokens")
class TokenEmbedding(Embedding):
    def __init__(self, spec, weights, runtime):
        self.spec, self.table = spec, weights[spec.table]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.table, (spec.vocab_size, spec.width), "table")]

    def forward(self, ctx, position):
        x = kernels.embed(ctx.token_ids, ctx.positions, self.table, position.embedding_table())
        return position.on_embedding(x, ctx)
