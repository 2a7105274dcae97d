from .base import (  # noqa: F401
    ConfigError, ModelConfig, build_spec, config_from_dict, known_architectures, load_config,
    lookup_architecture, register_architecture,
)
from .engine import EngineConfig, normalize_dtype  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
from .presets import load_preset, preset_names  # noqa: F401
