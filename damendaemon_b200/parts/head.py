"""Heads: from the residual stream to float32 logits at the wanted rows.

'linear': the final norm on the wanted rows only, then logits = y . W^T (+ bias); W may be the embedding's
table (damendaemon/gpt2.py:18,65-66: ``head is embed``, the norm after the last prompt row was picked).
"""
from __future__ import annotations

import torch

from .interfaces import Head
from .linear import linear
from .registry import NORMS, lookup, register_head
from .spec import TensorDecl


@register_head("linear")
class LinearHead(Head):
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.norm = lookup(NORMS, spec.norm, "norm")(spec.norm, weights, runtime)
        self.weight = weights[spec.weight]
        self.bias = weights[spec.bias] if spec.bias else None

    @staticmethod
    def tensor_decls(spec):
        decls = list(lookup(NORMS, spec.norm, "norm").tensor_decls(spec.norm))
        if not spec.tied:
            decls.append(TensorDecl(spec.weight, (spec.vocab_size, spec.width), "matrix"))
        if spec.bias:
            decls.append(TensorDecl(spec.bias, (spec.vocab_size,), "vector"))
        return decls

    def forward(self, x, ctx):
        y = self.norm.forward(x, row_index=ctx.want_rows)
        return linear(self.runtime, y, self.weight, self.bias, out_dtype=torch.float32)
