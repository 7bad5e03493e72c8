"""The one registry from an architecture's name to its configuration class.

``config.json["architectures"][0]`` selects the entry; everything that loads a
model folder (the Python entry point, the command line, trace replay, the bench)
goes through ``load_model_config``.  tinyserve dispatches on ``model_type`` with
``if`` switches inside one Model class (serve.py:70, 824, 831, 1305); here an
architecture is a configuration class whose ``model_spec()`` names the parts.
"""
from __future__ import annotations

import json
import os

from .babadra import BabadraConfig
from .delilorn import DelilornConfig
from .dudatar import DudatarConfig
from .model_config import ConfigError, ModelConfig, Qwen3Config
from .tarivik import TarivikConfig

ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    """Add (or replace) an architecture.  ``config_cls`` is a ModelConfig subclass."""
    if not (isinstance(config_cls, type) and issubclass(config_cls, ModelConfig)):
        raise TypeError("config_cls must be a ModelConfig subclass")
    ARCHITECTURES[name] = config_cls


def architecture_of(raw: dict) -> str:
    names = raw.get("architectures")
    if not names and isinstance(raw.get("architecture"), str):
        return raw["architecture"]           # some configurations name their one architecture plainly
    if not names or not isinstance(names, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list")
    return names[0]


def config_from_dict(raw: dict, model_dir: str = "") -> ModelConfig:
    """``model_dir``: the folder the configuration came from, for a configuration class that
    takes sizes from the shapes of the checkpoint's tensors (``reads_tensor_shapes``)."""
    name = architecture_of(raw)
    if name not in ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not registered; known: {sorted(ARCHITECTURES)}")
    cls = ARCHITECTURES[name]
    if getattr(cls, "reads_tensor_shapes", False):
        shapes = None
        if model_dir and any(f.endswith(".safetensors") for f in os.listdir(model_dir)):
            from ..weights.loader import tensor_shapes
            shapes = tensor_shapes(model_dir)
        return cls.from_dict(raw, shapes)
    return cls.from_dict(raw)


def load_model_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir!r} holds no config.json")
    with open(path) as fh:
        return config_from_dict(json.load(fh), model_dir)


register_architecture(Qwen3Config.architecture, Qwen3Config)
register_architecture(DudatarConfig.architecture, DudatarConfig)
register_architecture(DelilornConfig.architecture, DelilornConfig)
register_architecture(TarivikConfig.architecture, TarivikConfig)
register_architecture(BabadraConfig.architecture, BabadraConfig)
