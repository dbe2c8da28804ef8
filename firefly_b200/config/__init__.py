from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                   read_config_json)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "ScheduleEntry",
           "Qwen3Config", "read_config_json"]
