"""Configuration: typed per-architecture classes, the registry, and the model plan."""
from .plan import LayerSpec, ModelPlan, PartSpec, StreamStep
from .registry import (ConfigError, config_class_for, config_from_dict, known_architectures,
                       load_config, register_architecture)
from .qwen3 import Qwen3Config
from .dozazen import DozazenConfig
from .lagulorn import LagulornConfig
from .fagunex import FagunexConfig
from .fedinex import FedinexConfig

__all__ = ["LayerSpec", "ModelPlan", "PartSpec", "StreamStep", "ConfigError", "config_class_for", "config_from_dict",
           "known_architectures", "load_config", "register_architecture", "Qwen3Config", "DozazenConfig", "LagulornConfig",
           "FagunexConfig", "FedinexConfig"]
