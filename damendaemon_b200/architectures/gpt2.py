"""GPT-2 (``GPT2LMHeadModel``) described with the framework's parts.

Formulas and tensor names follow damendaemon/gpt2.py:8-66: learned absolute
positions (wte + wpe), pre-LayerNorm blocks, fused ``c_attn`` QKV stored as Conv1D
[in, out], full multi-head causal attention (key/value heads = heads), a gelu MLP,
``ln_f`` and an LM head tied to ``wte``.
"""
from __future__ import annotations

import math

import torch

from ..config.gpt2 import ARCHITECTURE, Gpt2Config
from ..parts.spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, NormSpec,
                          PositionSpec, RunEntry)
from ..registry import Architecture, register_architecture


def build_spec(c: Gpt2Config) -> ModelSpec:
    layers = []
    for i in range(c.n_layer):
        p = f"h.{i}."
        scale = c.head_dim ** -0.5
        if c.scale_attn_by_inverse_layer_idx:
            scale /= (i + 1)
        layers.append(LayerSpec(
            arrangement="pre_norm",
            norms=(NormSpec("layernorm", c.n_embd, c.layer_norm_epsilon, p + "ln_1.weight", p + "ln_1.bias"),
                   NormSpec("layernorm", c.n_embd, c.layer_norm_epsilon, p + "ln_2.weight", p + "ln_2.bias")),
            mixer=AttentionSpec("attention", width=c.n_embd, n_heads=c.n_head, n_kv_heads=c.n_head,
                                head_dim=c.head_dim, scale=scale, window=None,
                                qkv_weight=p + "attn.c_attn.weight", qkv_bias=p + "attn.c_attn.bias",
                                out_weight=p + "attn.c_proj.weight", out_bias=p + "attn.c_proj.bias",
                                stored_in_out=True),
            feed_forward=DenseFeedForwardSpec("dense", width=c.n_embd, inner=c.n_inner,
                                              activation=c.activation_function,
                                              up_weight=p + "mlp.c_fc.weight", up_bias=p + "mlp.c_fc.bias",
                                              down_weight=p + "mlp.c_proj.weight", down_bias=p + "mlp.c_proj.bias",
                                              stored_in_out=True),
        ))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=c.vocab_size, width=c.n_embd, max_positions=c.n_positions,
        embedding=EmbeddingSpec("tokens", c.vocab_size, c.n_embd, table="wte.weight"),
        position=PositionSpec("learned", c.n_positions, c.n_embd, table="wpe.weight"),
        layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(c.n_layer)),
        # the LM head is the token table (damendaemon/gpt2.py:18)
        head=HeadSpec("linear", c.vocab_size, c.n_embd,
                      norm=NormSpec("layernorm", c.n_embd, c.layer_norm_epsilon, "ln_f.weight", "ln_f.bias"),
                      weight="wte.weight", tied=True),
        eos_token_ids=tuple(c.eos_token_ids),
        # saved causal-mask buffers are not parameters (damendaemon/gpt2.py:26-28)
        ignored_tensors=(r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias"),
        tied_duplicates=(("lm_head.weight", "wte.weight"),),
        optional_prefix="transformer.",
    )


def random_tensors(c: Gpt2Config, seed: int, matrix_dtype=torch.float32, device="cpu") -> dict:
    """Seeded random GPT-2 weights under their checkpoint names, in a fixed draw order.

    Tables and matrices ~N(0, 0.02); both ``c_proj`` matrices ~N(0, 0.02/sqrt(2*n_layer));
    biases ~N(0, 0.02); LayerNorm gamma = 1 + N(0, 0.02), beta ~N(0, 0.02). Matrices and
    tables are stored in ``matrix_dtype``; vectors stay float32. ``device``: where the numbers
    are drawn (the CPU stream and a CUDA stream differ; a model folder is always written
    from the CPU stream).
    """
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    h, inner = c.n_embd, c.n_inner
    out = {}

    def normal(shape, std, mean=0.0):
        return torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std + mean

    def matrix(name, shape, std=0.02):
        out[name] = normal(shape, std).to(matrix_dtype)

    def vector(name, n, mean=0.0):
        out[name] = normal((n,), 0.02, mean)

    matrix("wte.weight", (c.vocab_size, h))
    matrix("wpe.weight", (c.n_positions, h))
    proj_std = 0.02 / math.sqrt(2 * c.n_layer)
    for i in range(c.n_layer):
        p = f"h.{i}."
        vector(p + "ln_1.weight", h, 1.0)
        vector(p + "ln_1.bias", h)
        matrix(p + "attn.c_attn.weight", (h, 3 * h))
        vector(p + "attn.c_attn.bias", 3 * h)
        matrix(p + "attn.c_proj.weight", (h, h), proj_std)
        vector(p + "attn.c_proj.bias", h)
        vector(p + "ln_2.weight", h, 1.0)
        vector(p + "ln_2.bias", h)
        matrix(p + "mlp.c_fc.weight", (h, inner))
        vector(p + "mlp.c_fc.bias", inner)
        matrix(p + "mlp.c_proj.weight", (inner, h), proj_std)
        vector(p + "mlp.c_proj.bias", h)
    vector("ln_f.weight", h, 1.0)
    vector("ln_f.bias", h)
    return out


register_architecture(Architecture(ARCHITECTURE, Gpt2Config.from_dict, build_spec, random_tensors), replace=True)
