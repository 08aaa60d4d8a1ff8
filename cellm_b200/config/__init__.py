from .errors import ConfigError
from .plan import PartSpec, LayerSpec, OrderEntry, ModelPlan
from .registry import (register_architecture, registered_architectures, resolve_architecture,
                       config_from_dict, load_config)
from .lfm2 import Lfm2Config
from .engine_config import EngineConfig, parse_dtype

__all__ = ["ConfigError", "PartSpec", "LayerSpec", "OrderEntry", "ModelPlan",
           "register_architecture", "registered_architectures", "resolve_architecture",
           "config_from_dict", "load_config", "Lfm2Config", "EngineConfig", "parse_dtype"]
