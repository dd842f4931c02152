from .base import (
    LayerCall,
    LayerSpec,
    ModelConfig,
    ModelSpec,
    PartSpec,
    UnsupportedConfigError,
    read_config_json,
)
from .registry import (
    config_class_for,
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
)

__all__ = [
    "LayerCall", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "UnsupportedConfigError",
    "read_config_json", "config_class_for", "config_from_dict", "known_architectures",
    "load_config", "register_architecture",
]
