from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .qwen2 import Qwen2Config
from .pufuzen import PufuzenConfig
from .katopel import KatopelConfig
from .vizonex import VizonexConfig
from .zobelorn import ZobelornConfig

__all__ = [
    "ConfigError", "KatopelConfig", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "PufuzenConfig", "Qwen2Config", "VizonexConfig", "ZobelornConfig",
    "config_class_for", "config_from_dict", "load_config", "register_architecture",
    "registered_architectures",
]
