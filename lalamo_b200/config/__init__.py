"""Typed configurations, part specifications and the architecture registry."""

from .errors import ConfigError, UnknownArchitectureError
from .lfm2 import Lfm2Config
from .plan import (
    AttentionSpec,
    BlockSpec,
    FeedForwardSpec,
    GatedMLPSpec,
    MixerSpec,
    ModelPlan,
    NormSpec,
    PositionSpec,
    RMSNormSpec,
    RopeSpec,
    ScheduleEntry,
    ShortConvSpec,
)
from .registry import architectures, config_from_dict, load_config, register_architecture

register_architecture("Lfm2ForCausalLM", Lfm2Config)

__all__ = [
    "AttentionSpec",
    "BlockSpec",
    "ConfigError",
    "FeedForwardSpec",
    "GatedMLPSpec",
    "Lfm2Config",
    "MixerSpec",
    "ModelPlan",
    "NormSpec",
    "PositionSpec",
    "RMSNormSpec",
    "RopeSpec",
    "ScheduleEntry",
    "ShortConvSpec",
    "UnknownArchitectureError",
    "architectures",
    "config_from_dict",
    "load_config",
    "register_architecture",
]
