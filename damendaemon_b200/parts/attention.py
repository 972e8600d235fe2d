"""The attention mixer: fused QKV projection, cache write, paged causal attention, output
projection with the residual add in its epilogue (damendaemon/gpt2.py:48-61).

Heads, key/value groups, head size, scale and window are parameters of the spec. The
kernels read keys and values from the cache pages only, so a portion of a prompt sees
earlier portions exactly as a decoded token sees its context.
"""
from __future__ import annotations

import torch

from ..cache.manager import PagedKeyValues
from .paged_attention import prompt_key_block
from .interfaces import Mixer
from .linear import linear
from .registry import register_mixer
from .spec import TensorDecl


def _joined(names):
    """The key of a tensor that the checkpoint holds whole (its name) or in pieces (their names joined)."""
    return names if isinstance(names, str) else "+".join(names)


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.qkv_w = weights[_joined(spec.qkv_weight)]
        self.qkv_b = weights[_joined(spec.qkv_bias)] if spec.qkv_bias else None
        self.out_w = weights[spec.out_weight]
        self.out_b = weights[spec.out_bias] if spec.out_bias else None
        self.q_width = spec.n_heads * spec.head_dim
        self.kv_width = spec.n_kv_heads * spec.head_dim
        if spec.head_dim % 8 or spec.head_dim > 256:
            raise ValueError(f"head size {spec.head_dim} is not supported (multiples of 8 up to 256)")
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads cannot share {spec.n_kv_heads} key/value heads")
        # where this mixer likes a prompt to be cut: the key block of its prompt kernel, if that kernel takes its sizes
        self.portion_multiple = 1
        if runtime.dtype == torch.bfloat16 and runtime.attention == "auto" and runtime.gemm != "simt":
            self.portion_multiple = prompt_key_block(spec.n_heads, spec.n_kv_heads, spec.head_dim, runtime.page_size, runtime.dtype)

    @staticmethod
    def tensor_decls(spec):
        q, kv = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        total = q + 2 * kv
        io = spec.stored_in_out
        matrix = lambda n: (spec.width, n) if io else (n, spec.width)
        # one fused projection in the checkpoint, or separate query, key and value projections joined at load
        pieces = () if isinstance(spec.qkv_weight, str) else tuple(zip(spec.qkv_weight, (matrix(q), matrix(kv), matrix(kv))))
        decls = [TensorDecl(_joined(spec.qkv_weight), matrix(total), "matrix", io, pieces),
                 TensorDecl(spec.out_weight, (q, spec.width) if io else (spec.width, q), "matrix", io)]
        if spec.qkv_bias:
            pieces = () if isinstance(spec.qkv_bias, str) else tuple(zip(spec.qkv_bias, ((q,), (kv,), (kv,))))
            decls.append(TensorDecl(_joined(spec.qkv_bias), (total,), "vector", False, pieces))
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
