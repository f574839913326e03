"""Typed configurations, the architecture registry and the neutral model description."""
from .base import (BlockSpec, ConfigError, ModelSpec, PartSpec, ScheduleEntry,
                   default_schedule)
from .llama import LlamaConfig, RopeScaling
from .registry import (config_from_dict, known_architectures, load_config,
                       lookup_architecture, preset_config, preset_names,
                       register_architecture, spec_from_config)

__all__ = ["BlockSpec", "ConfigError", "ModelSpec", "PartSpec", "ScheduleEntry",
           "default_schedule", "LlamaConfig", "RopeScaling", "config_from_dict",
           "known_architectures", "load_config", "lookup_architecture", "preset_config",
           "preset_names", "register_architecture", "spec_from_config"]
