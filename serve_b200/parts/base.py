"""Interfaces and registries of the parts a layer is put together from.

Five kinds of part exist: mixer (attention here), feed-forward, norm, position
encoding and block arrangement, plus the embedding and the output head that
bracket the layers. Each kind has a registry from a name to a class; a
``PartSpec`` (kind + params + tensor-name prefix) picks and parametrises one.
A part never looks at a model configuration: everything it needs is in its
params, and everything it runs goes through the kernels object it is given.

Adding a part means writing a class with the interface below and registering it
under a new name; the framework's files do not change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..config.spec import PartSpec


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part wants from the weight file.

    role: "matrix" is cast to the compute dtype (bfloat16 or float32);
          "vector" keeps 32-bit storage if the file has it, else the compute dtype;
          "table" is an integer table, kept as int32.
    init: how the random-weights mode fills it ("normal" or "norm").
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class CacheNeed:
    """What one execution of a mixer wants from the cache manager.

    A mixer with keys and values in pages gives kv_heads/head_dim (and a window
    if only the last ``window`` keys are ever read). A mixer with per-request
    state of fixed size gives ``state_shape`` (elements of float32 per request).
    Either may be absent.
    """

    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Optional[Tuple[int, ...]] = None

    @property
    def has_pages(self) -> bool:
        return self.kv_heads > 0 and self.head_dim > 0

    def group_key(self) -> Tuple:
        """Executions with equal keys share page geometry, a pool and block tables."""
        return (self.kv_heads, self.head_dim, self.window)


class Part:
    """Base of all parts. ``spec.params`` holds every size and constant."""

    def __init__(self, spec: PartSpec, runtime):
        self.spec = spec
        self.prefix = spec.prefix
        self.rt = runtime  # serve_b200.engine.runtime.Runtime: kernels, device, dtypes

    def tensor_decls(self) -> List[TensorDecl]:
        return []

    def ignorable_tensors(self) -> List[str]:
        """Names that may be in the file without being used (no 'unexpected' error)."""
        return []

    def load(self, tensors: Dict[str, Any]) -> None:
        """Take the declared tensors (already on the device, in their kept dtype)."""


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, h, ctx, cache):
        """h: [T, hidden] activations -> [T, hidden] activations (the residual delta).

        ``ctx`` is the step's StepContext; ``cache`` the CacheView of this
        execution (None if the mixer declared no need). ``cache.writes`` tells
        whether this execution owns the cache or only reads another's.
        """
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, ctx):
        raise NotImplementedError


class Norm(Part):
    def forward(self, x, delta, ctx):
        """x (float32 residual, updated in place with ``delta`` if given) -> normalised activations."""
        raise NotImplementedError

    def forward_rows(self, x, delta, rows, ctx):
        """As forward, but only for the rows listed (no update of x)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Held by a mixer; describes how positions enter queries and keys."""


class Block(Part):
    """An arrangement of parts around the residual stream.

    ``wants`` maps the names the arrangement gives its parts to their families
    ("mixer", "feed_forward", "norm", ...); the layer description brings one
    PartSpec per name, the constructor builds each and keeps it as an attribute of
    that name. ``spec.params`` holds the arrangement's own constants, if it has
    any. The part named "mixer", if there is one, is the one whose cache the
    layer owns; an arrangement whose cached part has another name overrides
    ``cache_need``.
    """

    wants: Dict[str, str] = {}

    def __init__(self, spec: PartSpec, runtime, parts: Optional[Dict[str, PartSpec]] = None):
        super().__init__(spec, runtime)
        given = dict(parts or {})
        missing = [n for n in self.wants if n not in given]
        extra = [n for n in given if n not in self.wants]
        if missing or extra:
            raise KeyError(f"block {spec.kind!r} arranges the parts {sorted(self.wants)}; the layer description "
                           f"lacks {sorted(missing)} and has {sorted(extra)} beyond them")
        self._built = []
        for name, family in self.wants.items():
            part = build_part(family, given[name], runtime)
            setattr(self, name, part)
            self._built.append(part)

    def parts(self) -> List[Part]:
        return list(self._built)

    def cache_need(self) -> Optional[CacheNeed]:
        mixer = getattr(self, "mixer", None)
        return mixer.cache_need() if mixer is not None else None

    def forward(self, x, pending, ctx, cache):
        """(x, pending) -> (x, pending); ``pending`` is a delta not yet added to x."""
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "block": {},
    "embedding": {},
    "head": {},
}


def register_part(family: str, name: str):
    """Class decorator: make a part constructible from ``PartSpec(kind=name)``."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r}; families: {', '.join(_REGISTRIES)}")

    def deco(cls):
        _REGISTRIES[family][name] = cls
        return cls

    return deco


def build_part(family: str, spec: PartSpec, runtime, **extra):
    try:
        cls = _REGISTRIES[family][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES.get(family, {}))) or "(none)"
        raise KeyError(f"no {family} part named {spec.kind!r}; registered: {known}") from None
    return cls(spec, runtime, **extra)


def registered(family: str) -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRIES[family]))
