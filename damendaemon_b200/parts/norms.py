"""Norms. LayerNorm with weight and optional bias (damendaemon/starcoder.py:53-55)."""
from __future__ import annotations

from .. import kernels
from .interfaces import Norm
from .registry import register_norm
from .spec import TensorDecl


@register_norm("layernorm")
class LayerNorm(Norm):
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.gamma = weights[spec.weight]
        self.beta = weights[spec.bias] if spec.bias else None

    @staticmethod
    def tensor_decls(spec):
        decls = [TensorDecl(spec.weight, (spec.width,), "vector")]
        if spec.bias:
            decls.append(TensorDecl(spec.bias, (spec.width,), "vector"))
        return decls

    def forward(self, x, row_index=None, out_dtype=None):
        return kernels.layernorm(x, self.gamma, self.beta, self.spec.eps, out_dtype or self.runtime.dtype, row_index)
