"""Configuration system: Configurable components, job sections, CLI/TOML manager, overrides."""

from .configurable import Configurable, ConfigRef, Function, config_to_dict
from .configs import (
    ActivationCheckpointConfig,
    CommConfig,
    CompileConfig,
    DebugConfig,
    KernelConfig,
    ModelSelectConfig,
    ParallelismConfig,
    TrainingConfig,
)
from .manager import ConfigError, ConfigManager, apply_dotted_overrides, apply_mapping
from .override import OverrideConfig, OverrideConflict, apply_overrides, derive, override

__all__ = [
    "Configurable", "ConfigRef", "config_to_dict", "Function",
    "ActivationCheckpointConfig", "CommConfig", "CompileConfig", "DebugConfig", "KernelConfig",
    "ModelSelectConfig", "ParallelismConfig", "TrainingConfig",
    "ConfigError", "ConfigManager", "apply_dotted_overrides", "apply_mapping",
    "OverrideConfig", "OverrideConflict", "apply_overrides", "derive", "override",
]
