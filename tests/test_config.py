"""Configuration parsing and the architecture registry (mirrors damendaemon tests/test_config.py:194-213)."""
import json

import pytest

from damendaemon_b200.config import ConfigError, Gpt2Config, parse_config_text, read_config_file
from damendaemon_b200.registry import architecture_of, load_config


def base():
    return {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 12, "n_embd": 768,
            "n_head": 12, "n_positions": 1024, "vocab_size": 50257, "activation_function": "gelu_new"}


def test_dimension_mapping():
    c = Gpt2Config.from_dict(base())
    assert (c.head_dim, c.n_inner, c.layer_norm_epsilon) == (64, 3072, 1e-5)
    assert Gpt2Config.from_dict({**base(), "n_inner": 1024}).n_inner == 1024
    assert Gpt2Config.from_dict({**base(), "n_inner": None}).n_inner == 3072
    assert Gpt2Config.from_dict({**base(), "activation_function": "gelu"}).activation_function == "gelu"
    assert Gpt2Config.from_dict({**base(), "scale_attn_by_inverse_layer_idx": True}).scale_attn_by_inverse_layer_idx
    assert Gpt2Config.from_dict({**base(), "eos_token_id": 50256}).eos_token_ids == (50256,)


@pytest.mark.parametrize("change", [
    {"architectures": ["GPT2Model"]}, {"architectures": None}, {"model_type": "llama"},
    {"n_layer": 0}, {"n_embd": "768"}, {"n_head": 7}, {"n_embd": 36, "n_head": 12}, {"n_inner": True}, {"n_inner": -4},
    {"layer_norm_epsilon": 0}, {"layer_norm_epsilon": -1e-5}, {"activation_function": "relu"},
    {"scale_attn_weights": False}, {"tie_word_embeddings": False}, {"add_cross_attention": True},
    {"reorder_and_upcast_attn": True}, {"quantization_config": {"bits": 4}}, {"vocab_size": None},
    {"eos_token_id": 50257}, {"scale_attn_by_inverse_layer_idx": 1},
])
def test_rejected_variants(change):
    with pytest.raises(ConfigError):
        Gpt2Config.from_dict({**base(), **change})


def test_round_trip(tiny_configs):
    for raw in tiny_configs.values():
        c = Gpt2Config.from_dict(raw)
        assert Gpt2Config.from_dict(c.to_dict()) == c


def test_reader_rules(tmp_path):
    with pytest.raises(ConfigError, match="duplicate"):
        parse_config_text(b'{"a": 1, "a": 2}')
    for bad in (b'{"a": NaN}', b'{"a": Infinity}', b'{"a": 1e999}', b'[1]', b'\xff\xfe', b'{"a":'):
        with pytest.raises(ConfigError):
            parse_config_text(bad)
    with pytest.raises(ConfigError, match="1 MiB"):
        parse_config_text(b'{"a": "' + b"x" * (1024 * 1024) + b'"}')
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_file(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(base()))
    arch, typed = load_config(tmp_path)
    assert arch.name == "GPT2LMHeadModel" and typed.n_layer == 12


def test_registry_errors():
    with pytest.raises(ConfigError, match="unknown architecture"):
        architecture_of({"architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="exactly one"):
        architecture_of({"architectures": ["A", "B"]})


def test_spec_has_no_hidden_sizes(tiny_configs):
    """Every size in the spec comes from the configuration."""
    arch = architecture_of(tiny_configs["B"])
    c = arch.parse_config(tiny_configs["B"])
    spec = arch.build_spec(c)
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    m = spec.layers[2].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.window) == (2, 2, 48, None)
    assert m.scale == pytest.approx(48 ** -0.5 / 3)
    assert spec.layers[0].feed_forward.inner == 320 and spec.layers[0].feed_forward.activation == "gelu"
    assert spec.head.norm.eps == 1e-6 and spec.position.n_positions == 256
