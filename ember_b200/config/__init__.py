"""Typed configurations and the architecture registry."""
from .spec import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec, ModelSpec, NoPositionSpec,
                   PartSpec, RMSNormSpec, RotarySpec, ScheduleEntry, default_schedule)
from .registry import (config_from_dict, load_config, load_model_spec, register_architecture,
                       registered_architectures, resolve_architecture)
from .qwen3 import Qwen3Config

__all__ = [
    "AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NoPositionSpec", "PartSpec",
    "RMSNormSpec", "RotarySpec", "ScheduleEntry", "default_schedule", "config_from_dict", "load_config",
    "load_model_spec", "register_architecture", "registered_architectures", "resolve_architecture",
    "Qwen3Config",
]
