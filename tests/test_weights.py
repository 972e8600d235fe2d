"""Weight loading by name: prefixes, ignored buffers, the tied head, and ONE error that lists
everything that is wrong (mirrors the corruptions of the reference's
tests/test_starcoder_cpu_reference.py and tests/test_floating_parameter.py:46-63)."""
import json

import pytest
import torch

from conftest import TINY_A, TINY_B
from damendaemon_b200.parts import tensor_decls
from damendaemon_b200.registry import architecture_of
from damendaemon_b200.weights import (CheckpointFormatError, DictSource, SafetensorsFile, WeightError, check_and_place,
                                      load_weights, write_random_model, write_safetensors)


def setup(config):
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    spec = arch.build_spec(typed)
    return arch, typed, spec, tensor_decls(spec)


def test_random_folder_round_trip(tmp_path):
    arch, typed, spec, decls = setup(TINY_B)
    folder = write_random_model(tmp_path / "m", TINY_B, seed=1, dtype="bfloat16")
    again = write_random_model(tmp_path / "n", TINY_B, seed=1, dtype="bfloat16")
    assert (folder / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    other = write_random_model(tmp_path / "o", TINY_B, seed=2, dtype="bfloat16")
    assert (folder / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()
    assert json.loads((folder / "config.json").read_text())["n_inner"] == 320
    with SafetensorsFile(folder / "model.safetensors") as f:
        assert f.describe("wte.weight") == (torch.bfloat16, (1000, 96))
        assert f.describe("h.0.ln_1.weight") == (torch.float32, (96,))
        assert f.describe("h.2.mlp.c_fc.weight") == (torch.bfloat16, (96, 320))
    for engine_dtype in (torch.bfloat16, torch.float32):
        w = load_weights(folder, spec, decls, engine_dtype, "cpu")
        assert w["h.1.attn.c_attn.weight"].shape == (288, 96) and w["h.1.attn.c_attn.weight"].dtype == engine_dtype
        assert w["h.1.attn.c_attn.weight"].is_contiguous()
        assert w["h.1.mlp.c_proj.weight"].shape == (96, 320)
        assert w["h.1.attn.c_attn.bias"].dtype == torch.float32 and w["ln_f.weight"].dtype == torch.float32
        assert w["wpe.weight"].dtype == engine_dtype
    # the init scheme: c_proj matrices are narrower by sqrt(2 * n_layer)
    t = arch.random_tensors(typed, 1)
    assert t["h.0.attn.c_proj.weight"].std() < 0.6 * t["h.0.attn.c_attn.weight"].std()
    assert abs(float(t["h.0.ln_1.weight"].mean()) - 1.0) < 0.02


def test_prefix_buffers_and_tied_head():
    arch, typed, spec, decls = setup(TINY_A)
    t = arch.random_tensors(typed, 0)
    plain = check_and_place(DictSource(t), spec, decls, torch.float32, "cpu")
    prefixed = {"transformer." + k: v for k, v in t.items()}
    prefixed["transformer.h.0.attn.bias"] = torch.ones(1, 1, 128, 128)
    prefixed["transformer.h.1.attn.masked_bias"] = torch.tensor(-1e4)
    prefixed["lm_head.weight"] = t["wte.weight"].clone()
    placed = check_and_place(DictSource(prefixed), spec, decls, torch.float32, "cpu")
    assert all(torch.equal(plain[k], placed[k]) for k in plain)
    prefixed["lm_head.weight"] = t["wte.weight"] + 1
    with pytest.raises(WeightError, match="tied"):
        check_and_place(DictSource(prefixed), spec, decls, torch.float32, "cpu")


def test_one_error_lists_everything():
    arch, typed, spec, decls = setup(TINY_A)
    t = arch.random_tensors(typed, 0)
    del t["h.1.ln_2.bias"], t["wpe.weight"]
    t["h.0.mlp.c_fc.weight"] = t["h.0.mlp.c_fc.weight"].t().contiguous()      # [out, in] instead of Conv1D's [in, out]
    t["h.0.attn.c_proj.bias"] = torch.zeros(63)
    t["h.0.extra.weight"] = torch.zeros(2)
    t["ln_f.weight"] = torch.ones(64, dtype=torch.int8)
    with pytest.raises(WeightError) as info:
        check_and_place(DictSource(t), spec, decls, torch.float32, "cpu")
    e = info.value
    assert sorted(e.missing) == ["h.1.ln_2.bias", "wpe.weight"] and e.unexpected == ["h.0.extra.weight"]
    assert len(e.wrong_shape) == 2 and len(e.wrong_dtype) == 1
    text = str(e)
    for piece in ("missing tensors (2)", "h.1.ln_2.bias", "unexpected tensors (1)", "h.0.extra.weight", "wrong shapes (2)",
                  "expected (64, 256), found (256, 64)", "wrong dtypes (1)", "ln_f.weight"):
        assert piece in text, piece


def test_file_format_checks(tmp_path):
    path = tmp_path / "model.safetensors"
    write_safetensors(path, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.zeros(0)})
    with SafetensorsFile(path) as f:
        assert f.tensor("a").tolist() == [[0, 1, 2], [3, 4, 5]] and f.tensor("b").numel() == 0
    raw = path.read_bytes()
    path.write_bytes(raw[:-4])
    with pytest.raises(CheckpointFormatError):
        SafetensorsFile(path)
    path.write_bytes(b"\xff" * 8 + raw[8:])
    with pytest.raises(CheckpointFormatError, match="header length"):
        SafetensorsFile(path)
    path.write_bytes(raw[:8] + raw[8:].replace(b'"a"', b'"b"', 1))
    with pytest.raises(CheckpointFormatError, match="duplicate"):
        SafetensorsFile(path)
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(tmp_path / "nowhere", None, [], torch.float32, "cpu")


def test_engine_refuses_without_cuda(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("needs a machine without CUDA")
    from damendaemon_b200.engine import Engine
    from damendaemon_b200.kernels import KernelError
    folder = write_random_model(tmp_path / "m", TINY_A, 0)
    with pytest.raises(KernelError, match="no CPU fallback"):
        Engine(folder, dtype="float32")


def test_sharded_checkpoint(tmp_path):
    arch, typed, spec, decls = setup(TINY_A)
    t = arch.random_tensors(typed, 0)
    names = sorted(t)
    half = len(names) // 2
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: t[n] for n in names[:half]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: t[n] for n in names[half:]})
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    sharded = load_weights(tmp_path, spec, decls, torch.float32, "cpu")
    whole = check_and_place(DictSource(t), spec, decls, torch.float32, "cpu")
    assert all(torch.equal(sharded[k], whole[k]) for k in whole)
    (tmp_path / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightError, match="shards"):
        load_weights(tmp_path, spec, decls, torch.float32, "cpu")


def test_tensors_stored_in_pieces_are_joined_at_load(tmp_path):
    """Separate query, key and value projections in the checkpoint (stored [in, out] here, and with grouped key/value
    heads so that the three differ in width) become the one fused matrix the attention mixer reads; a missing or
    misshapen piece is named in the one error."""
    import torch
    from damendaemon_b200.parts import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec,
                                        NormSpec, PositionSpec, RunEntry, tensor_decls)
    from damendaemon_b200.weights import DictSource, WeightError, check_and_place
    width, heads, kv_heads, d = 32, 4, 2, 8
    norm = lambda n: NormSpec("layernorm", width, 1e-5, n + ".weight", n + ".bias")
    mixer = AttentionSpec("attention", width, heads, kv_heads, d, d ** -0.5, None,
                          qkv_weight=("q.weight", "k.weight", "v.weight"), qkv_bias=("q.bias", "k.bias", "v.bias"),
                          out_weight="o.weight", out_bias=None, stored_in_out=True)
    ff = DenseFeedForwardSpec("dense", width, 64, "gelu_new", "up.weight", None, "down.weight", None)
    spec = ModelSpec("Pieces", 50, width, 16, EmbeddingSpec("tokens", 50, width, "embed.weight"), PositionSpec("none", 16, width),
                     (LayerSpec("pre_norm", mixer, ff, (norm("n1"), norm("n2"))),), (RunEntry(0),),
                     HeadSpec("linear", 50, width, norm("nf"), "head.weight"))
    decls = tensor_decls(spec)
    joined = next(d_ for d_ in decls if d_.name == "q.weight+k.weight+v.weight")
    assert joined.shape == (width, 64) and [n for n, _ in joined.pieces] == ["q.weight", "k.weight", "v.weight"]
    g = torch.Generator().manual_seed(0)
    tensors = {}
    for d_ in decls:
        for name, shape in (d_.pieces or ((d_.name, d_.shape),)):
            tensors[name] = torch.randn(shape, generator=g)
    placed = check_and_place(DictSource(tensors), spec, decls, torch.float32, "cpu")
    fused = placed["q.weight+k.weight+v.weight"]
    assert fused.shape == (64, width) and fused.is_contiguous()
    assert torch.equal(fused, torch.cat([tensors["q.weight"].t(), tensors["k.weight"].t(), tensors["v.weight"].t()]))
    assert torch.equal(placed["q.bias+k.bias+v.bias"], torch.cat([tensors["q.bias"], tensors["k.bias"], tensors["v.bias"]]))
    assert "head.weight" in placed and placed["head.weight"].shape == (50, width)       # an untied head has its own matrix
    broken = dict(tensors)
    del broken["k.weight"]
    broken["v.bias"] = torch.zeros(9)
    broken["q.weight+k.weight+v.weight"] = torch.zeros(width, 64)
    with pytest.raises(WeightError) as info:
        check_and_place(DictSource(broken), spec, decls, torch.float32, "cpu")
    assert info.value.missing == ["k.weight"] and info.value.unexpected == ["q.weight+k.weight+v.weight"]
    assert any(w.startswith("v.bias") for w in info.value.wrong_shape)
