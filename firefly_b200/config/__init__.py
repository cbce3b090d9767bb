from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                   read_config_json)
from .kefisun import KefisunConfig
from .kolorax import KoloraxConfig
from .papusun import PapusunConfig
from .pepolorn import PepolornConfig
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "ScheduleEntry",
           "KefisunConfig", "KoloraxConfig", "PapusunConfig", "PepolornConfig", "Qwen3Config", "read_config_json"]
