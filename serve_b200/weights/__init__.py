from .loader import WeightError, load_from_source, load_weights  # noqa: F401
from .random_init import random_tensor, write_random_model  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
