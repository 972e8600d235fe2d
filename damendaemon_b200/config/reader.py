"""Bounded, strict reading of a model folder's ``config.json``.

Same rules as the reference's ``read_config`` (damendaemon/config.py:10-50):
at most 1 MiB, UTF-8, one JSON object, no duplicate keys, no NaN/Infinity.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

MAX_CONFIG_BYTES = 1024 * 1024


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the field."""


def _unique(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            raise ConfigError(f"config.json: duplicate field {key!r}")
        seen[key] = value
    return seen


def _finite(text):
    value = float(text)
    if not math.isfinite(value):
        raise ConfigError("config.json: non-finite number")
    return value


def _no_constant(name):
    raise ConfigError(f"config.json: non-finite constant {name}")


def parse_config_text(raw: bytes) -> dict:
    if len(raw) > MAX_CONFIG_BYTES:
        raise ConfigError("config.json exceeds 1 MiB")
    try:
        text = raw.decode("utf-8")
    except UnicodeDecodeError as error:
        raise ConfigError("config.json is not UTF-8") from error
    try:
        value = json.loads(text, object_pairs_hook=_unique, parse_float=_finite,
                           parse_constant=_no_constant)
    except RecursionError as error:
        raise ConfigError("config.json nesting is too deep") from error
    except json.JSONDecodeError as error:
        raise ConfigError(f"config.json is not valid JSON: {error}") from error
    if not isinstance(value, dict):
        raise ConfigError("config.json must hold one JSON object")
    return value


def read_config_file(path) -> dict:
    """Read ``path`` (a config.json, or a folder that holds one)."""
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json at {path}")
    with path.open("rb") as reader:
        raw = reader.read(MAX_CONFIG_BYTES + 1)
    return parse_config_text(raw)
