from .base import ConfigError, KeyReader, ModelConfig, read_config_json
from .dabodra import DabodraConfig
from .llama import LlamaConfig, RopeScaling
from .mokatar import MokatarConfig
from .nibelorn import NibelornConfig
from .vitinex import VitinexConfig
from .registry import (Architecture, architecture_name, find_architecture, register_architecture,
                       registered_architectures)

__all__ = ["ConfigError", "KeyReader", "ModelConfig", "read_config_json", "LlamaConfig", "RopeScaling", "NibelornConfig", "DabodraConfig", "VitinexConfig", "MokatarConfig",
           "Architecture", "architecture_name", "find_architecture", "register_architecture",
           "registered_architectures"]
