from . import qwen2  # noqa: F401  (registers the architecture)
from .model import DecoderModel
from .registry import Architecture, architecture_of, get_architecture, read_model_config, register_architecture

__all__ = ["DecoderModel", "Architecture", "architecture_of", "get_architecture", "read_model_config", "register_architecture"]
