"""Feed-forwards. Dense two-matrix MLP with the activation fused into the first product's
epilogue and the residual add into the second's (damendaemon/gpt2.py:62-64)."""
from __future__ import annotations

from .interfaces import FeedForward
from .linear import linear
from .registry import register_feed_forward
from .spec import TensorDecl

ACTIVATIONS = ("gelu_new", "gelu")


@register_feed_forward("dense")
class DenseFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not supported; known: {ACTIVATIONS}")
        self.spec, self.runtime = spec, runtime
        self.up_w, self.down_w = weights[spec.up_weight], weights[spec.down_weight]
        self.up_b = weights[spec.up_bias] if spec.up_bias else None
        self.down_b = weights[spec.down_bias] if spec.down_bias else None

    @staticmethod
    def tensor_decls(spec):
        io = spec.stored_in_out
        decls = [TensorDecl(spec.up_weight, (spec.width, spec.inner) if io else (spec.inner, spec.width), "matrix", io),
                 TensorDecl(spec.down_weight, (spec.inner, spec.width) if io else (spec.width, spec.inner), "matrix", io)]
        if spec.up_bias:
            decls.append(TensorDecl(spec.up_bias, (spec.inner,), "vector"))
        if spec.down_bias:
            decls.append(TensorDecl(spec.down_bias, (spec.width,), "vector"))
        return decls

    def forward(self, y, residual, ctx):
        hidden = linear(self.runtime, y, self.up_w, self.up_b, activation=self.spec.activation)
        return linear(self.runtime, hidden, self.down_w, self.down_b, residual=residual, out_dtype=residual.dtype,
                      out=residual)
