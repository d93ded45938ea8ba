from .goguvik import GoguvikConfig
from .qwen3 import ConfigError, Qwen3Config
from .registry import ARCHITECTURES, config_from_dict, load_config, register_architecture
from .spec import (
    AttentionSpec,
    DifferentialAttentionSpec,
    DynamicTanhSpec,
    GatedFeedForwardSpec,
    HyperConnectionSpec,
    LayerSpec,
    ModelSpec,
    NormSpec,
    QueryTemperatureSpec,
    RopeSpec,
    ScheduleEntry,
    default_schedule,
    hyper_layer,
    prenorm_layer,
)

__all__ = [
    "ARCHITECTURES",
    "AttentionSpec",
    "ConfigError",
    "DifferentialAttentionSpec",
    "DynamicTanhSpec",
    "GatedFeedForwardSpec",
    "GoguvikConfig",
    "HyperConnectionSpec",
    "QueryTemperatureSpec",
    "hyper_layer",
    "LayerSpec",
    "ModelSpec",
    "NormSpec",
    "Qwen3Config",
    "RopeSpec",
    "ScheduleEntry",
    "config_from_dict",
    "default_schedule",
    "load_config",
    "prenorm_layer",
    "register_architecture",
]
