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
    """One block: its arrangement and the parts it is made of, by role.

    ``parts`` maps a role of the arrangement ("mixer", "mixer_norm", "feed_forward", "ff_norm" for
    the pre-norm block; another arrangement names its own roles and may have more or fewer) to the
    part that fills it; ``names`` maps each role to its sub-prefix in the checkpoint, e.g.
    mixer -> "self_attn".  A role without a name uses the role itself as sub-prefix.
    """

    prefix: str
    block: str
    parts: tuple[tuple[str, PartSpec], ...]
    names: tuple[tuple[str, str], ...] = ()

    @staticmethod
    def make(prefix: str, block: str, parts: Mapping[str, PartSpec],
             names: Mapping[str, str] | None = None) -> "LayerSpec":
        return LayerSpec(prefix, block, tuple(parts.items()), tuple((names or {}).items()))

    @staticmethod
    def pre_norm(prefix: str, *, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec,
                 ff_norm: PartSpec, names: Mapping[str, str] | None = None) -> "LayerSpec":
        """The pre-norm block with Hugging Face's sub-prefixes unless ``names`` gives others."""
        default = {"mixer": "self_attn", "mixer_norm": "input_layernorm", "feed_forward": "mlp",
                   "ff_norm": "post_attention_layernorm"}
        return LayerSpec.make(prefix, "pre_norm",
                              {"mixer_norm": mixer_norm, "mixer": mixer, "ff_norm": ff_norm,
                               "feed_forward": feed_forward}, {**default, **(names or {})})

    def part(self, role: str) -> PartSpec:
        for r, spec in self.parts:
            if r == role:
                return spec
        known = ", ".join(r for r, _ in self.parts)
        raise KeyError(f"layer {self.prefix!r} has no part in the role {role!r}; it has: {known}")

    def roles(self) -> tuple[str, ...]:
        return tuple(r for r, _ in self.parts)

    def name_of(self, role: str) -> str:
        return dict(self.names).get(role, role)


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
class PagedNeed(CacheNeed):
    """Per-position memory in pages.  A subclass says what one page looks like.

    ``window``: None keeps every position; a number keeps the last ``window`` positions, and pages
    that the window has passed are given back.  Entries whose needs compare equal share one
    group: one pool, one allocator, one block table per request.  So a need holds what decides
    the memory's geometry and lifetime and nothing else: how a mixer's kernels tile their work is
    the mixer's business (its planner), not a reason for a pool of its own.
    """

    kind: str = field(default="pages", init=False)
    window = None          # a subclass makes this a field if its mixer can have a window

    def page_shape(self, page_size: int) -> tuple[int, ...]:
        """Shape of one page of one cache entry for pages of ``page_size`` positions."""
        raise NotImplementedError


@dataclass(frozen=True)
class PagedKVNeed(PagedNeed):
    """Keys and values of every cached position: a page is [2 (K, V), kv_heads, page_size, head_dim]."""

    kv_heads: int = 1
    head_dim: int = 16
    window: int | None = None

    def page_shape(self, page_size: int) -> tuple[int, ...]:
        return (2, self.kv_heads, page_size, self.head_dim)


@dataclass(frozen=True)
class StateNeed(CacheNeed):
    """A fixed-size state per request (recurrent state, a running sum, ...), zero at admission."""

    shape: tuple[int, ...]
    dtype: str = "float32"
    kind: str = field(default="state", init=False)
