"""Random-weights mode: write a model folder from a configuration and a seed."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..registry import architecture_of
from .safetensors_io import write_safetensors

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def write_random_model(folder, config: dict, seed: int, dtype="float32", name_prefix="") -> Path:
    """Create ``folder`` with config.json and model.safetensors; returns the folder.

    ``config`` holds the architecture's own config.json keys. ``dtype`` is how matrices
    and tables are stored (vectors are stored in float32). ``name_prefix`` (for example
    'transformer.') is put before every tensor name.
    """
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    tensors = arch.random_tensors(typed, seed, _DTYPES[dtype] if isinstance(dtype, str) else dtype)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    with (folder / "config.json").open("w") as f:
        json.dump(typed.to_dict(), f, indent=1)
    write_safetensors(folder / "model.safetensors", {name_prefix + k: v for k, v in tensors.items()},
                      {"format": "pt", "seed": seed})
    return folder
