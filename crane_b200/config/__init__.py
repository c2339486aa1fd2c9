"""Typed configurations and the architecture registry."""
from .hunyuan_dense import (ALIASES, ARCHITECTURE, ConfigError, HunyuanDenseConfig, RopeScaling,
                            build_spec, read_config_json)
from .registry import (Architecture, UnknownArchitecture, register_architecture, registered,
                       resolve)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep
from .engine_config import EngineConfig, parse_memory_limit

register_architecture(ARCHITECTURE, HunyuanDenseConfig.from_dict, build_spec, ALIASES)

__all__ = ["ConfigError", "HunyuanDenseConfig", "RopeScaling", "read_config_json", "Architecture",
           "UnknownArchitecture", "register_architecture", "registered", "resolve", "LayerSpec",
           "ModelSpec", "PartSpec", "ScheduleStep", "EngineConfig", "parse_memory_limit"]
