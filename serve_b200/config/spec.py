"""The layer-by-layer description of a model, as plain data.

An architecture's builder turns its typed configuration into a ``ModelSpec``:
which part (mixer, feed-forward, norm, position encoding) sits in which layer,
with every size and constant as a parameter of that part, and the order in
which layers run. Nothing below the builder knows which model it is part of.

The reference wires one fixed block N times (serve/model.py:137-160); here the
wiring is data so that layers may differ, a layer may run twice, and a layer
may read the cache that another one wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` is its registry key, ``params`` its constructor arguments."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    # prefix of this part's tensor names in the weight file, e.g. "model.layers.3.self_attn."
    prefix: str = ""

    def with_prefix(self, prefix: str) -> "PartSpec":
        return PartSpec(self.kind, dict(self.params), prefix)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement (a part with parameters of its own) and the parts it arranges, by the
    names the arrangement gives them. Which names an arrangement wants, and of which family each is, the
    arrangement's class says (``Block.wants``): "pre_norm" wants mixer, feed_forward, mixer_norm and
    feed_forward_norm; an arrangement with other norms, without a feed-forward or with two mixers side by side
    names other parts, and nothing else changes."""

    block: PartSpec
    parts: Dict[str, PartSpec]

    @classmethod
    def pre_norm(cls, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec) -> "LayerSpec":
        """The reference's arrangement (serve/model.py:146-149)."""
        return cls(PartSpec("pre_norm"), {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": mixer_norm,
                                          "feed_forward_norm": feed_forward_norm})


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` (an index may appear more than once:
    the weights are shared, each execution has a cache of its own).
    ``cache_of`` names an earlier schedule entry whose cache this execution
    reads instead of writing one itself; None means it owns its cache.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    max_position: int

    def validate(self) -> None:
        from .base import ConfigError

        if not self.schedule:
            raise ConfigError("a model needs at least one scheduled layer")
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which owns none")
