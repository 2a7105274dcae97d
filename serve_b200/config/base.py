"""Architecture registry and the base of every typed model configuration.

A model folder's ``config.json`` names its architecture in ``architectures[0]``.
The registry maps that name to two things: the typed configuration class that
reads the file's keys, and a function that turns such a configuration into a
``ModelSpec`` (the layer-by-layer description the engine builds parts from).

The reference keys its hyper-parameters on hub repository names
(serve/utils.py:35-38) and picks a dict by name suffix
(serve/hf_utils/convert_hf_checkpoint.py:62-65); here the file itself decides.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple, Type


class ConfigError(ValueError):
    """A configuration file is missing a key, or holds a value this engine refuses."""


@dataclass(frozen=True)
class ModelConfig:
    """Base class of typed architecture configurations."""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":  # pragma: no cover - interface
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:  # pragma: no cover - interface
        raise NotImplementedError


# architecture name -> (config class, spec builder)
_ARCHITECTURES: Dict[str, Tuple[Type[ModelConfig], Callable[[Any], Any]]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], build_spec: Callable[[Any], Any]) -> None:
    """Make ``name`` (as it appears in config.json ``architectures``) loadable."""
    _ARCHITECTURES[name] = (config_cls, build_spec)


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def lookup_architecture(name: str) -> Tuple[Type[ModelConfig], Callable[[Any], Any]]:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; this engine knows: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def architecture_of(d: Dict[str, Any]) -> str:
    archs = d.get("architectures")
    if not isinstance(archs, (list, tuple)) or len(archs) == 0 or not isinstance(archs[0], str):
        raise ConfigError("config.json needs a non-empty 'architectures' list naming the model class")
    return archs[0]


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    """Typed configuration from parsed config.json content, chosen by its architecture."""
    config_cls, _ = lookup_architecture(architecture_of(d))
    return config_cls.from_dict(d)


def load_config(model_dir: str) -> ModelConfig:
    """Read ``model_dir/config.json`` into the typed configuration of its architecture."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)


def build_spec(config: ModelConfig):
    """The ``ModelSpec`` of a typed configuration (through the registry)."""
    for _name, (config_cls, builder) in _ARCHITECTURES.items():
        if type(config) is config_cls:
            return builder(config)
    raise ConfigError(f"no architecture registered for configuration type {type(config).__name__}")
