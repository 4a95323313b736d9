"""Typed configurations and the architecture registry."""
from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry, read_config_json)
from .banitar import BanitarConfig
from .fiferax import FiferaxConfig
from .gemma2 import Gemma2Config
from .tarorax import TaroraxConfig
from .zatasun import ZatasunConfig
from .registry import (architecture_name, config_from_dict, config_from_folder,
                       known_architectures, register_architecture)

register_architecture(Gemma2Config.architecture, Gemma2Config)
register_architecture(FiferaxConfig.architecture, FiferaxConfig)
register_architecture(BanitarConfig.architecture, BanitarConfig)
register_architecture(ZatasunConfig.architecture, ZatasunConfig)
register_architecture(TaroraxConfig.architecture, TaroraxConfig)

__all__ = [
    "ConfigError", "KeyReader", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "ScheduleEntry",
    "read_config_json", "BanitarConfig", "FiferaxConfig", "Gemma2Config", "TaroraxConfig", "ZatasunConfig", "architecture_name", "config_from_dict",
    "config_from_folder", "known_architectures", "register_architecture",
]
