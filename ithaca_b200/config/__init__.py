from .base import ConfigError, load_config_dict
from .gunenex import GunenexConfig
from .llama import LlamaConfig, RopeScaling
from .mimadra import MimadraConfig
from .tiralix import TiralixConfig
from .vebisun import VebisunConfig
from .registry import (Architecture, config_from_dict, config_from_model_dir, lookup_architecture,
                       register_architecture, registered_architectures, unregister_architecture)
from .spec import (BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule, describe,
                   validate_schedule)

__all__ = [
    "ConfigError", "LlamaConfig", "VebisunConfig", "TiralixConfig", "MimadraConfig", "GunenexConfig", "RopeScaling", "load_config_dict", "Architecture", "config_from_dict",
    "config_from_model_dir", "lookup_architecture", "register_architecture", "registered_architectures",
    "unregister_architecture", "BlockSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule",
    "describe", "validate_schedule",
]
