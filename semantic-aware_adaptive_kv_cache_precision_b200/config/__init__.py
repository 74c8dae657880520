"""Typed configurations and the architecture registry."""

from .specs import (AttentionSpec, BlockSpec, ConfigError, GatedMLPSpec, LayerCall, ModelSpec,
                    NormSpec, RotarySpec)
from .registry import (architecture_name, config_from_dict, config_from_folder,
                       known_architectures, register_architecture)
from .qwen2 import Qwen2Config

__all__ = ["AttentionSpec", "BlockSpec", "ConfigError", "GatedMLPSpec", "LayerCall", "ModelSpec",
           "NormSpec", "RotarySpec", "Qwen2Config", "architecture_name", "config_from_dict",
           "config_from_folder", "known_architectures", "register_architecture"]
