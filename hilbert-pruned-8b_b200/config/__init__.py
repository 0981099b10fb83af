from .base import ConfigError, read_config_json
from .llama import Llama3RopeScaling, LlamaConfig
from .registry import (config_class_for, load_config, register_architecture, registered_architectures,
                       unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

__all__ = ["ConfigError", "Llama3RopeScaling", "LlamaConfig", "read_config_json", "config_class_for",
           "load_config", "register_architecture", "registered_architectures", "unregister_architecture",
           "LayerSpec", "ModelSpec", "PartSpec", "PlanEntry"]

register_architecture(LlamaConfig)
