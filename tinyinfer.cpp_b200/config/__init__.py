"""Typed configurations, the architecture registry and the architecture-independent plan."""
from .plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry, default_schedule
from .registry import (Architecture, ConfigError, architecture_of, get_architecture,
                       known_architectures, load_config, read_config_json,
                       register_architecture)
from .qwen3 import Qwen3Config

__all__ = [
    "Architecture", "ConfigError", "LayerPlan", "ModelPlan", "PartSpec", "Qwen3Config",
    "ScheduleEntry", "architecture_of", "default_schedule", "get_architecture",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
]
