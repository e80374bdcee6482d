from . import qwen3  # registers the architecture
from .decoder import DecoderModel

__all__ = ["DecoderModel", "qwen3"]
