"""Tiny random model folders for the tests (made in temporary folders, never committed)."""
import json
from pathlib import Path

import torch

from damendaemon_b200.registry import architecture_of
from damendaemon_b200.weights import write_safetensors


def make_model(folder, config, seed, dtype="float32", sharpen=8.0):
    """Random weights, with the QKV projection scaled up so that attention is not nearly
    uniform (with N(0, 0.02) weights every key weighs about the same and a wrong key,
    a missing key or a stale page would barely move the logits)."""
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    store = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    tensors = arch.random_tensors(typed, seed, torch.float32)
    for name in tensors:
        if name.endswith("attn.c_attn.weight"):
            tensors[name] = tensors[name] * sharpen
        if tensors[name].dim() == 2:
            tensors[name] = tensors[name].to(store)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(typed.to_dict()))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def random_requests(config, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, config["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
