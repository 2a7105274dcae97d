"""Named configurations (JSON files beside this module) for the random-weights mode."""
from __future__ import annotations

import json
import os

from ..base import ConfigError, config_from_dict

_DIR = os.path.dirname(os.path.abspath(__file__))


def preset_names():
    return tuple(sorted(f[:-5] for f in os.listdir(_DIR) if f.endswith(".json")))


def load_preset(name: str):
    path = os.path.join(_DIR, name + ".json")
    if not os.path.isfile(path):
        raise ConfigError(f"no preset {name!r}; presets: {', '.join(preset_names())}")
    with open(path) as f:
        return config_from_dict(json.load(f))
