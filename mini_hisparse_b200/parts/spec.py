"""Data that describes a model: which parts each layer is made of, and in which order layers run.

A model class turns its typed configuration into a :class:`ModelSpec`; everything below the
spec (parts, cache manager, step function, loader) is generic and never asks which model it
serves.  The reference hard-wires one block type (mini_hisparse/model.py:74-88); here the
block's parts are chosen layer by layer, and the run order is a list that may name a layer
twice or let an entry read the cache of an earlier entry.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """A part's kind (its name in the registry) and its sizes and constants."""

    kind: str
    params: tuple[tuple[str, Any], ...] = ()

    @staticmethod
    def make(kind: str, **params) -> "PartSpec":
        return PartSpec(kind, tuple(sorted(params.items())))

    def __getitem__(self, key: str):
        for k, v in self.params:
            if k == key:
                return v
        raise KeyError(f"part {self.kind!r} has no parameter {key!r}")

    def get(self, key: str, default=None):
        for k, v in self.params:
            if k == key:
                return v
        return default

    def as_dict(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class ParamSpec:
    """One stored tensor of a part.

    role: "matrix" tensors take the compute dtype (bfloat16 when serving, float32 on the
    32-bit path); "vector" tensors (norm weights, biases) are always held in float32, so one
    stored in 32-bit stays so; "table" tensors are integer tables held as int32.
    init: how the random-weights mode draws it: ("normal", mean, std).
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: tuple = ("normal", 0.0, 0.02)
    optional: bool = False


@dataclass(frozen=True)
class LayerSpec:
    """One block: its arrangement and the four parts it is made of.

    ``names`` maps each part to its sub-prefix in the checkpoint, e.g. mixer -> "self_attn".
    """

    prefix: str
    block: str
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    ff_norm: PartSpec
    names: tuple[tuple[str, str], ...] = (
        ("mixer", "self_attn"),
        ("mixer_norm", "input_layernorm"),
        ("feed_forward", "mlp"),
        ("ff_norm", "post_attention_layernorm"),
    )

    def name_of(self, part: str) -> str:
        return dict(self.names)[part]


@dataclass(frozen=True)
class RunEntry:
    """One step of the run order: which layer's weights run, and whose cache it uses.

    ``cache_of`` is None when the entry owns a cache of its own (it appends to it), or the
    index of an EARLIER entry of the run order whose cache this entry only reads.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    embedding_name: str
    layers: tuple[LayerSpec, ...]
    order: tuple[RunEntry, ...]
    final_norm: PartSpec
    final_norm_name: str
    head: PartSpec
    head_name: str
    max_positions: int | None = None
    eos_token_id: int | None = None

    def __post_init__(self):
        for i, e in enumerate(self.order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run entry {i} names layer {e.layer}, but there are {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"run entry {i} reads the cache of entry {e.cache_of}, which is not earlier")
                if self.order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run entry {i} reads entry {e.cache_of}, which owns no cache")


# ---- what a mixer needs from the cache manager ---------------------------------------------

@dataclass(frozen=True)
class CacheNeed:
    """Base of the two kinds of per-request memory a mixer can ask for."""


@dataclass(frozen=True)
class PagedKVNeed(CacheNeed):
    """Keys and values of every cached position, in pages.

    ``window``: None keeps all keys; a number keeps the last ``window`` keys, and pages that the
    window has passed are given back.  Layers whose needs compare equal share one group: one
    pool, one block table per request.
    """

    kv_heads: int
    head_dim: int
    q_heads: int
    window: int | None = None
    tile_rows: int = 16      # query rows per attention tile for long portions (a kernel's choice)
    kind: str = field(default="pages", init=False)


@dataclass(frozen=True)
class StateNeed(CacheNeed):
    """A fixed-size state per request (recurrent state, a running sum, ...), zero at admission."""

    shape: tuple[int, ...]
    dtype: str = "float32"
    kind: str = field(default="state", init=False)
