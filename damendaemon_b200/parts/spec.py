"""Declarative description of a decoder: what each part is and how layers are arranged.

An architecture turns its typed configuration into one ``ModelSpec``. Every size
and constant a part needs is a field of its spec, so no part knows which model it
is in; ``kind`` selects the implementation from the part registries, layer by
layer, so one model may mix different mixers and feed-forwards. The order in
which layers run is data as well (``run_order``): an entry may name a layer twice
or let a layer read another layer's cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One checkpoint tensor a part wants.

    role: 'matrix' and 'table' are kept in the engine dtype (bfloat16 or float32),
    'vector' is always float32 (biases, norm parameters), 'int' is int32.
    ``stored_in_out``: the checkpoint holds the matrix as [in, out] (GPT-2 Conv1D);
    the device copy is always [out, in], K-contiguous.
    ``pieces``: the checkpoint does not hold this tensor whole but as several tensors
    ((checkpoint name, shape as stored), ...) that are joined along the output axis, in
    this order, when they are placed (separate query, key and value projections that one
    fused product reads); ``name`` is then only the key under which the part finds the
    joined tensor, and ``shape`` its shape as if it had been stored whole.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    stored_in_out: bool = False
    pieces: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()


@dataclass(frozen=True)
class NormSpec:
    kind: str            # 'layernorm'
    width: int
    eps: float
    weight: str          # checkpoint names
    bias: Optional[str] = None


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # 'learned'
    n_positions: int
    width: int
    table: Optional[str] = None


@dataclass(frozen=True)
class AttentionSpec:
    kind: str            # 'attention'
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float         # multiplies q.k (already includes any per-layer factor)
    window: Optional[int]  # None = all earlier keys; n = the query and the n-1 keys before it
    qkv_weight: object   # checkpoint name of the fused projection, or the three names (query, key, value) of separate ones
    qkv_bias: object     # None, one name, or three names
    out_weight: str
    out_bias: Optional[str]
    stored_in_out: bool = False


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    kind: str            # 'dense'
    width: int
    inner: int
    activation: str      # 'gelu_new' | 'gelu'
    up_weight: str
    up_bias: Optional[str]
    down_weight: str
    down_bias: Optional[str]
    stored_in_out: bool = False


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a mixer, a feed-forward, as many norms as its arrangement wants, and the arrangement that wires them
    ('pre_norm' takes two norms: before the mixer, before the feed-forward)."""
    arrangement: str
    mixer: object
    feed_forward: object
    norms: Tuple[object, ...]

    @property
    def kind(self):
        return self.arrangement


@dataclass(frozen=True)
class EmbeddingSpec:
    kind: str            # 'tokens': a row of the table per token id (the position encoding may add its own table)
    vocab_size: int
    width: int
    table: str           # checkpoint name


@dataclass(frozen=True)
class HeadSpec:
    kind: str            # 'linear': final norm on the wanted rows, then logits = y . W^T (+ bias)
    vocab_size: int
    width: int
    norm: object         # a norm spec
    weight: str          # checkpoint name of W [vocab, width]
    tied: bool = False   # W is the embedding's table (declared there, not again)
    bias: Optional[str] = None


@dataclass(frozen=True)
class RunEntry:
    """One stop of the forward pass: run ``layer`` (an index into ``ModelSpec.layers``).

    Every stop has a cache of its own, so a layer that is named twice keeps the keys and
    values of its two runs apart. ``cache_of`` = the index of an EARLIER STOP in
    ``run_order`` makes this stop read that stop's cache instead: it gets no pages of its
    own and does not write (its mixer sees ``cache.writable == False``).
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: object                 # an embedding spec
    position: object                  # a position-encoding spec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    head: object                      # a head spec (with the final norm)
    eos_token_ids: Tuple[int, ...] = ()
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)   # regexes of tensors to drop
    tied_duplicates: Tuple[Tuple[str, str], ...] = field(default_factory=tuple)  # (name, must equal)
    optional_prefix: str = ""          # e.g. 'transformer.': stripped from every name when present

    @property
    def prefix_probe(self):
        """The tensor whose presence under the optional prefix says that the checkpoint uses the prefix."""
        return self.embedding.table
