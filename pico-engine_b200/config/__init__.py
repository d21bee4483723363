"""Typed configurations, part descriptions and the architecture registry."""
from .specs import (ConfigError, PartSpec, RMSNormSpec, RotaryHalfSpec, NoPositionSpec, GQAAttentionSpec,
                    SwiGLUSpec, LayerSpec, ScheduleEntry, ModelPlan)
from .registry import (Architecture, register_architecture, known_architectures, architecture,
                       architecture_name_of, config_from_dict, read_config)
from .qwen2 import Qwen2Config

__all__ = ["ConfigError", "PartSpec", "RMSNormSpec", "RotaryHalfSpec", "NoPositionSpec", "GQAAttentionSpec",
           "SwiGLUSpec", "LayerSpec", "ScheduleEntry", "ModelPlan", "Architecture", "register_architecture",
           "known_architectures", "architecture", "architecture_name_of", "config_from_dict", "read_config",
           "Qwen2Config"]
