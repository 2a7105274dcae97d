"""Architectures: importing this package registers them."""
from . import llama  # noqa: F401
from .decoder import DecoderModel  # noqa: F401
