from .base import (Architecture, ConfigError, ModelConfig, architecture_of, load_config,
                   register_architecture, registered_architectures)
from .banevik import BanevikConfig
from .gemma2 import Gemma2Config
from .kedasun import KedasunConfig
from .neburax import NeburaxConfig
from .ritirax import RitiraxConfig

__all__ = ["Architecture", "ConfigError", "ModelConfig", "Gemma2Config", "BanevikConfig", "NeburaxConfig", "KedasunConfig", "RitiraxConfig", "architecture_of",
           "load_config", "register_architecture", "registered_architectures"]
