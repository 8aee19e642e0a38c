"""Configuration: model specification, architecture registry, engine sizes."""

from .engine_config import EngineConfig, parse_dtype
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .basitar import BasitarConfig
from .kopatar import KopatarConfig
from .mezadra import MezadraConfig
from .qwen3 import Qwen3Config
from .zupupel import ZupupelConfig
from .registry import (
    load_config,
    read_config_json,
    register_architecture,
    resolve_architecture,
    supported_architectures,
)

register_architecture(Qwen3Config)
register_architecture(KopatarConfig)
register_architecture(MezadraConfig)
register_architecture(BasitarConfig)
register_architecture(ZupupelConfig)

__all__ = [
    "BasitarConfig",
    "EngineConfig",
    "KopatarConfig",
    "LayerSpec",
    "MezadraConfig",
    "ModelSpec",
    "PartSpec",
    "Qwen3Config",
    "ScheduleEntry",
    "ZupupelConfig",
    "load_config",
    "parse_dtype",
    "read_config_json",
    "register_architecture",
    "resolve_architecture",
    "supported_architectures",
]
