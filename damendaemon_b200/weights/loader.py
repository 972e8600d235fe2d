"""Load a model folder's tensors by name, check them against what the model's parts declare.

Every part lists the checkpoint tensors it wants (``TensorDecl``: name, shape, role).
The loader reads ``model.safetensors``, strips the architecture's optional name
prefix, drops buffers the architecture says to ignore, and raises ONE error that
lists every missing tensor, every unexpected tensor, every wrong shape and every
non-floating dtype (the reference raises a bare KeyError on the first missing name,
damendaemon/gpt2.py:12-15,38; a named error is friendlier).

Dtypes on the device: 'matrix' and 'table' tensors are kept in the engine dtype
(bfloat16 for the serving path; a folder that stores them in 32-bit is rounded once
here), 'vector' tensors (biases, norm parameters) are always float32, 'int' tensors
int32. With the float32 engine everything floating is float32: a true 32-bit path.
Matrices stored [in, out] (GPT-2's Conv1D) are transposed once to [out, in], the
K-contiguous layout every GEMM kernel here reads (the reference transposes them at
load as well, damendaemon/gpt2.py:15,35).
"""
from __future__ import annotations

import re
from pathlib import Path

import torch

from ..parts.spec import TensorDecl
from .safetensors_io import SafetensorsFile

_FLOATING = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), unequal=()):
        super().__init__(message)
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype, self.unequal = list(wrong_shape), list(wrong_dtype), list(unequal)


def weight_files(model_dir) -> list:
    """``model.safetensors``, or the shards that ``model.safetensors.index.json`` names (every shard the index
    lists must exist; the reference cross-checks its index the same way, damendaemon/checkpoint.py:29-68)."""
    folder = Path(model_dir)
    single = folder / "model.safetensors"
    if single.is_file():
        return [single]
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        import json
        try:
            names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        except (ValueError, KeyError, AttributeError, TypeError) as error:
            raise WeightError(f"unreadable {index.name}: {error}") from error
        shards = [folder / n for n in names]
        gone = [p.name for p in shards if not p.is_file() or p.parent != folder]
        if gone or not shards:
            raise WeightError(f"{index.name} names shards that are not in {model_dir}: {gone}")
        return shards
    raise WeightError(f"no model.safetensors in {model_dir}")


def weight_file(model_dir) -> Path:
    return weight_files(model_dir)[0]


class ShardedSource:
    """Several safetensors files read as one; a tensor name may appear in one shard only."""

    def __init__(self, files):
        self.files = files
        self.where = {}
        for f in files:
            for name in f.names():
                if name in self.where:
                    raise WeightError(f"tensor {name} appears in two shards")
                self.where[name] = f

    def names(self):
        return list(self.where)

    def describe(self, name):
        return self.where[name].describe(name)

    def tensor(self, name):
        return self.where[name].tensor(name)


def check_and_place(source, spec, decls, engine_dtype, device):
    """``source``: an object with names()/describe(name)/tensor(name). Returns {name: device tensor}."""
    names = list(source.names())
    prefix = spec.optional_prefix
    strip = bool(prefix) and any(n.startswith(prefix) for n in names) and \
        (prefix + spec.prefix_probe) in names
    rename = {(n[len(prefix):] if strip and n.startswith(prefix) else n): n for n in names}
    ignored = [re.compile(p) for p in spec.ignored_tensors]
    # what the checkpoint must hold: every declared tensor, or its pieces where it is stored in pieces
    wanted = {}
    for d in decls:
        if d.pieces:
            for piece_name, piece_shape in d.pieces:
                wanted[piece_name] = TensorDecl(piece_name, tuple(piece_shape), d.role, d.stored_in_out)
        else:
            wanted[d.name] = d
    duplicates = dict(spec.tied_duplicates)

    missing = [n for n in wanted if n not in rename]
    unexpected, wrong_shape, wrong_dtype, unequal = [], [], [], []
    for short, full in rename.items():
        if short in wanted:
            decl = wanted[short]
            dtype, shape = source.describe(full)
            if tuple(shape) != tuple(decl.shape):
                wrong_shape.append(f"{short}: expected {tuple(decl.shape)}, found {tuple(shape)}")
            if decl.role == "int":
                if dtype.is_floating_point or dtype == torch.bool:
                    wrong_dtype.append(f"{short}: expected an integer tensor, found {dtype}")
            elif dtype not in _FLOATING:
                wrong_dtype.append(f"{short}: expected a floating tensor, found {dtype}")
        elif short in duplicates:
            pass
        elif any(p.fullmatch(short) for p in ignored):
            pass
        else:
            unexpected.append(short)
    for short, same_as in duplicates.items():
        if short in rename and same_as in rename and same_as not in [w.split(":")[0] for w in wrong_shape]:
            if source.describe(rename[short]) != source.describe(rename[same_as]) or \
                    not torch.equal(source.tensor(rename[short]), source.tensor(rename[same_as])):
                unequal.append(f"{short} differs from {same_as} although the two are tied")
    if missing or unexpected or wrong_shape or wrong_dtype or unequal:
        parts = []
        for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                             ("wrong shapes", wrong_shape), ("wrong dtypes", wrong_dtype),
                             ("unequal tied tensors", unequal)):
            if items:
                parts.append(f"{title} ({len(items)}): " + "; ".join(sorted(items)))
        raise WeightError(f"checkpoint does not fit {spec.architecture}: " + " | ".join(parts),
                          missing, unexpected, wrong_shape, wrong_dtype, unequal)

    placed = {}
    for decl in decls:
        if decl.pieces:
            # joined along the output axis: rows of the [out, in] device copy, the only axis of a vector
            parts = [source.tensor(rename[n]) for n, _ in decl.pieces]
            t = torch.cat([p.t() if decl.stored_in_out and p.dim() == 2 else p for p in parts], dim=0)
            if tuple(t.shape) != (tuple(reversed(decl.shape)) if decl.stored_in_out and len(decl.shape) == 2 else tuple(decl.shape)):
                raise ValueError(f"the pieces of {decl.name} do not add up to {tuple(decl.shape)}")
        else:
            t = source.tensor(rename[decl.name])
            if decl.role in ("matrix", "table") and decl.stored_in_out:
                t = t.t()
        if decl.role in ("matrix", "table"):
            t = t.to(device=device, dtype=engine_dtype).contiguous()
        elif decl.role == "vector":
            t = t.to(device=device, dtype=torch.float32).contiguous()
        elif decl.role == "int":
            t = t.to(device=device, dtype=torch.int32).contiguous()
        else:
            raise ValueError(f"unknown tensor role {decl.role!r} for {decl.name}")
        placed[decl.name] = t
    return placed


class DictSource:
    """Tensors already in memory (random weights that never touched the disk)."""

    def __init__(self, tensors: dict):
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def describe(self, name):
        t = self.tensors[name]
        return t.dtype, tuple(t.shape)

    def tensor(self, name):
        return self.tensors[name]


def load_weights(model_dir, spec, decls, engine_dtype, device):
    files = [SafetensorsFile(p) for p in weight_files(model_dir)]
    try:
        source = files[0] if len(files) == 1 else ShardedSource(files)
        return check_and_place(source, spec, decls, engine_dtype, device)
    finally:
        for f in files:
            f.close()
