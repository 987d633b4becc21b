"""Typed configurations and the architecture registry."""
from .registry import (config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .specs import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, RopeSpec, ScheduleEntry, SwiGLUSpec)
from .qwen3 import Qwen3Config

__all__ = ["config_class_for", "config_from_dict", "load_config", "register_architecture",
           "registered_architectures", "AttentionSpec", "BlockSpec", "ModelSpec", "NormSpec",
           "RopeSpec", "ScheduleEntry", "SwiGLUSpec", "Qwen3Config"]
