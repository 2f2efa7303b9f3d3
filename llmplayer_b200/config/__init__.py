"""Typed configurations and the architecture registry."""
from .registry import (
    ArchitectureConfig, config_class_for, config_from_dict, known_architectures, load_config,
    register_architecture, unregister_architecture,
)
from .llama import LlamaConfig
from .ramupel import RamupelConfig
from .botuvik import BotuvikConfig
from .zasitar import ZasitarConfig
from .dopuvik import DopuvikConfig

__all__ = [
    "ArchitectureConfig", "BotuvikConfig", "DopuvikConfig", "LlamaConfig", "RamupelConfig", "ZasitarConfig", "config_class_for", "config_from_dict",
    "known_architectures", "load_config", "register_architecture", "unregister_architecture",
]
