from .model_config import (ConfigError, LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                           Qwen3Config)
from .dudatar import DudatarConfig
from .delilorn import DelilornConfig
from .tarivik import TarivikConfig
from .babadra import BabadraConfig
from .registry import (ARCHITECTURES, architecture_of, config_from_dict, load_model_config,
                       register_architecture)
from .engine_config import EngineConfig

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec",
           "Qwen3Config", "DudatarConfig", "DelilornConfig", "TarivikConfig", "BabadraConfig", "ARCHITECTURES", "architecture_of", "config_from_dict",
           "load_model_config", "register_architecture", "EngineConfig"]
