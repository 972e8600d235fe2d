"""Typed GPT-2 configuration, parsed from the architecture's own config.json keys.

Field rules follow the reference's ``gpt2_config`` (damendaemon/config.py:299-320).
Two options the reference rejects are accepted here because the formulas are
simple and the tiny test configurations use them: ``activation_function='gelu'``
(exact erf form) and ``scale_attn_by_inverse_layer_idx=true`` (scores divided by
layer index + 1).
"""
from __future__ import annotations

import math
import sys
from dataclasses import dataclass

from .reader import ConfigError

ARCHITECTURE = "GPT2LMHeadModel"
ACTIVATIONS = ("gelu_new", "gelu")


def _positive_int(config, name):
    value = config.get(name)
    if type(value) is not int or value <= 0:
        raise ConfigError(f"{name} must be a positive integer, got {value!r}")
    return value


def _flag(config, name, default):
    value = config.get(name, default)
    if type(value) is not bool:
        raise ConfigError(f"{name} must be true or false, got {value!r}")
    return value


@dataclass(frozen=True)
class Gpt2Config:
    n_layer: int
    n_embd: int
    n_head: int
    n_inner: int
    n_positions: int
    vocab_size: int
    layer_norm_epsilon: float
    activation_function: str
    scale_attn_by_inverse_layer_idx: bool
    eos_token_ids: tuple = ()

    architecture = ARCHITECTURE

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @classmethod
    def from_dict(cls, config: dict) -> "Gpt2Config":
        if config.get("architectures") != [ARCHITECTURE]:
            raise ConfigError(f"architectures must be ['{ARCHITECTURE}'], got {config.get('architectures')!r}")
        if config.get("model_type", "gpt2") != "gpt2":
            raise ConfigError(f"model_type must be 'gpt2', got {config.get('model_type')!r}")
        sizes = {name: _positive_int(config, name)
                 for name in ("n_layer", "n_embd", "n_head", "n_positions", "vocab_size")}
        if sizes["n_embd"] % sizes["n_head"]:
            raise ConfigError("n_embd must be a multiple of n_head")
        if (sizes["n_embd"] // sizes["n_head"]) % 2:
            raise ConfigError("head size (n_embd / n_head) must be even")
        inner = config.get("n_inner")
        if inner is None:
            inner = 4 * sizes["n_embd"]
        if type(inner) is not int or inner <= 0:
            raise ConfigError(f"n_inner must be null or a positive integer, got {inner!r}")
        epsilon = config.get("layer_norm_epsilon", 1e-5)
        if type(epsilon) not in (int, float) or not 0 < epsilon <= sys.float_info.max or not math.isfinite(epsilon):
            raise ConfigError(f"layer_norm_epsilon must be finite and positive, got {epsilon!r}")
        activation = config.get("activation_function", "gelu_new")
        if activation not in ACTIVATIONS:
            raise ConfigError(f"activation_function must be one of {ACTIVATIONS}, got {activation!r}")
        if not _flag(config, "scale_attn_weights", True):
            raise ConfigError("scale_attn_weights=false is not supported")
        if not _flag(config, "tie_word_embeddings", True):
            raise ConfigError("tie_word_embeddings=false is not supported (the LM head is wte)")
        for name in ("add_cross_attention", "reorder_and_upcast_attn"):
            if _flag(config, name, False):
                raise ConfigError(f"{name}=true is not supported")
        if config.get("quantization_config"):
            raise ConfigError("quantized checkpoints are not supported")
        eos = config.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        for token in eos:
            if type(token) is not int or not 0 <= token < sizes["vocab_size"]:
                raise ConfigError(f"eos_token_id {token!r} is outside the vocabulary")
        return cls(n_inner=inner, layer_norm_epsilon=float(epsilon), activation_function=activation,
                   scale_attn_by_inverse_layer_idx=_flag(config, "scale_attn_by_inverse_layer_idx", False),
                   eos_token_ids=eos, **sizes)

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        out = {
            "architectures": [ARCHITECTURE], "model_type": "gpt2",
            "n_layer": self.n_layer, "n_embd": self.n_embd, "n_head": self.n_head,
            "n_inner": self.n_inner, "n_positions": self.n_positions, "vocab_size": self.vocab_size,
            "layer_norm_epsilon": self.layer_norm_epsilon,
            "activation_function": self.activation_function,
            "scale_attn_weights": True,
            "scale_attn_by_inverse_layer_idx": self.scale_attn_by_inverse_layer_idx,
            "tie_word_embeddings": True,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return out
