from . import kudazen, mirovik, nunivik, qwen2, tobadra  # noqa: F401  (register the architectures)
from .model import DecoderModel
from .registry import Architecture, architecture_of, get_architecture, read_model_config, register_architecture

__all__ = ["DecoderModel", "Architecture", "architecture_of", "get_architecture", "read_model_config", "register_architecture"]
