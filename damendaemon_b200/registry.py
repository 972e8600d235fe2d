"""The one registry from an architecture's name to its configuration and model.

``config.json``'s ``architectures[0]`` selects the entry everywhere in the framework
(engine, command line, trace replay, random-weights writer). The reference
dispatches on ``model_type`` in three places (damendaemon/config.py:119-145,
damendaemon/runtime.py:675-679, damendaemon/qwen2.py:195-196); here it is one table.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .config.reader import ConfigError, read_config_file


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable      # dict -> typed config
    build_spec: Callable        # typed config -> ModelSpec
    random_tensors: Callable    # (typed config, seed, matrix dtype) -> {checkpoint name: tensor}


ARCHITECTURES: dict = {}


def register_architecture(entry: Architecture, *, replace=False):
    if entry.name in ARCHITECTURES and not replace:
        raise ValueError(f"architecture {entry.name!r} is already registered")
    ARCHITECTURES[entry.name] = entry
    return entry


def architecture_of(config: dict) -> Architecture:
    names = config.get("architectures")
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError(f"config.json 'architectures' must name exactly one architecture, got {names!r}")
    _load_builtin()
    if names[0] not in ARCHITECTURES:
        raise ConfigError(f"unknown architecture {names[0]!r}; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[names[0]]


def load_config(model_dir):
    """Folder -> (Architecture, typed config)."""
    raw = read_config_file(model_dir)
    arch = architecture_of(raw)
    return arch, arch.parse_config(raw)


def _load_builtin():
    from .architectures import gpt2  # noqa: F401  (registers itself on import)
