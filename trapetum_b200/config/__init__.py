from .base import (ArchitectureEntry, ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, architecture,
                   architecture_name, known_architectures, load_config, read_config_dict, register_architecture)
from .divanex import DivanexConfig
from .fibelix import FibelixConfig
from .fidepel import FidepelConfig
from .gemma2 import Gemma2Config
from .lofirax import LofiraxConfig

__all__ = ["ArchitectureEntry", "ConfigError", "DivanexConfig", "FibelixConfig", "FidepelConfig", "Gemma2Config", "LayerSpec", "LofiraxConfig", "ModelSpec", "PartSpec", "ScheduleEntry",
           "architecture", "architecture_name", "known_architectures", "load_config", "read_config_dict",
           "register_architecture"]
