"""The attention mixer: fused QKV projection, cache write, paged causal attention, output
projection with the residual add in its epilogue (damendaemon/gpt2.py:48-61).

Heads, key/value groups, head size, scale and window are parameters of the spec. The
kernels read keys and values from the cache pages only, so a portion of a prompt sees
earlier portions exactly as a decoded token sees its context.
"""
from __future__ import annotations

from ..cache.manager import PagedKeyValues
from .interfaces import Mixer
from .linear import linear
from .registry import register_mixer
from .spec import TensorDecl


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.qkv_w = weights[spec.qkv_weight]
        self.qkv_b = weights[spec.qkv_bias] if spec.qkv_bias else None
        self.out_w = weights[spec.out_weight]
        self.out_b = weights[spec.out_bias] if spec.out_bias else None
        self.q_width = spec.n_heads * spec.head_dim
        self.kv_width = spec.n_kv_heads * spec.head_dim
        if spec.head_dim % 8 or spec.head_dim > 256:
            raise ValueError(f"head size {spec.head_dim} is not supported (multiples of 8 up to 256)")
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads cannot share {spec.n_kv_heads} key/value heads")

    @staticmethod
    def tensor_decls(spec):
        total = (spec.n_heads + 2 * spec.n_kv_heads) * spec.head_dim
        decls = [TensorDecl(spec.qkv_weight, (spec.width, total) if spec.stored_in_out else (total, spec.width),
                            "matrix", spec.stored_in_out),
                 TensorDecl(spec.out_weight, (spec.n_heads * spec.head_dim, spec.width) if spec.stored_in_out
                            else (spec.width, spec.n_heads * spec.head_dim), "matrix", spec.stored_in_out)]
        if spec.qkv_bias:
            decls.append(TensorDecl(spec.qkv_bias, (total,), "vector"))
        if spec.out_bias:
            decls.append(TensorDecl(spec.out_bias, (spec.width,), "vector"))
        return decls

    @staticmethod
    def cache_needs(spec):
        return [PagedKeyValues(spec.n_kv_heads, spec.head_dim, spec.window)]

    def forward(self, y, residual, ctx, cache, position):
        s = self.spec
        qkv = linear(self.runtime, y, self.qkv_w, self.qkv_b)
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        q, k = position.on_query_key(q, k, ctx)
        attended = ctx.attend(q, k, v, cache, s.n_heads, s.scale, s.window)
        return linear(self.runtime, attended, self.out_w, self.out_b, residual=residual, out_dtype=residual.dtype,
                      out=residual)
