from .base import ConfigError, ConfigReader, read_json
from .generation import GenerationDefaults, read_generation_defaults
from .kudazen import KudazenConfig
from .mirovik import MirovikConfig
from .nunivik import NunivikConfig
from .qwen2 import Qwen2Config
from .tobadra import TobadraConfig

__all__ = ["ConfigError", "ConfigReader", "read_json", "GenerationDefaults", "read_generation_defaults", "Qwen2Config", "NunivikConfig", "MirovikConfig", "KudazenConfig", "TobadraConfig"]
