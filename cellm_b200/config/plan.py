"""Architecture-neutral description of a model: which parts make each layer,
which tensors they read, and in which order the layers run.

An architecture's plan builder turns its typed configuration into a
`ModelPlan`. Everything below the plan (parts, cache manager, step function)
sees only the plan, never the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind, its sizes and constants, and
    the file tensor that backs each of its weights (local name -> file name)."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    weights: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: an arrangement (`block`) of a mixer, a feed-forward and their norms."""
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class OrderEntry:
    """One item of the run order. `layer` indexes `ModelPlan.layers`; the same
    layer may appear more than once (each appearance has a cache of its own).
    `cache_of`, if set, is the index in the order of an earlier item whose
    cache this item reads instead of writing one."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    """`embedding` and `head` are parts like the others (families "embedding" and "head"). For the usual pair, a
    table look-up and a plain output product, a file tensor's name may be given in their place: `embedding` the
    table [vocab, hidden]; `head` the output matrix [vocab, hidden], or None for one tied to the embedding."""
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: Any                      # PartSpec, or the name of the table's file tensor
    final_norm: PartSpec
    head: Any                           # PartSpec, or the name of the matrix' file tensor, or None (tied)
    layers: tuple[LayerSpec, ...]
    order: tuple[OrderEntry, ...]
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None

    def __post_init__(self):
        sizes = {"vocab_size": self.vocab_size, "dim": self.hidden_size}
        if isinstance(self.embedding, str):
            object.__setattr__(self, "embedding", PartSpec("lookup", dict(sizes), {"weight": self.embedding}))
        if self.head is None or isinstance(self.head, str):
            name = self.head if self.head is not None else self.embedding.weights.get("weight")
            object.__setattr__(self, "head", PartSpec("linear", dict(sizes), {"weight": name}))

    @property
    def tied(self) -> bool:
        """Whether the head reads the embedding's tensor."""
        return self.head.weights.get("weight") == self.embedding.weights.get("weight")

    def validate(self) -> None:
        from .errors import ConfigError
        for i, e in enumerate(self.order):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"layer order item {i} names layer {e.layer}, "
                                  f"but the model has {len(self.layers)} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ConfigError(f"layer order item {i} reads the cache of item {e.cache_of}, "
                                      f"which does not come before it")
                if self.order[e.cache_of].cache_of is not None:
                    raise ConfigError(f"layer order item {i} reads the cache of item {e.cache_of}, "
                                      f"which has no cache of its own")
