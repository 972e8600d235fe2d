"""Position encodings. Learned absolute positions: a table added to the token embedding
(damendaemon/gpt2.py:46); the add is fused into the embedding kernel."""
from __future__ import annotations

from .interfaces import PositionEncoding
from .registry import register_position
from .spec import TensorDecl


@register_position("learned")
class LearnedPositions(PositionEncoding):
    def __init__(self, spec, weights, runtime):
        self.spec = spec
        self.table = weights[spec.table]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.table, (spec.n_positions, spec.width), "table")]

    def embedding_table(self):
        return self.table


@register_position("none")
class NoPositions(PositionEncoding):
    def __init__(self, spec, weights, runtime):
        self.spec = spec
