"""Architectures.  Importing this package registers every one of them."""
from . import desarax, gegepel, qwen3, titatar, tosivik  # noqa: F401
from .decoder import DecoderModel, LayerCall

__all__ = ["DecoderModel", "LayerCall"]
