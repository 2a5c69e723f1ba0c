from .files import ConfigError, read_config_files
from .llama import Llama3RopeScaling, LlamaConfig
from .recipe import LayerSpec, ModelRecipe, PartSpec, Run
from .registry import Architecture, register_architecture, registered_architectures, resolve_architecture
from .engine import EngineConfig

__all__ = [
    "Architecture", "ConfigError", "EngineConfig", "LayerSpec", "Llama3RopeScaling", "LlamaConfig",
    "ModelRecipe", "PartSpec", "Run", "read_config_files", "register_architecture",
    "registered_architectures", "resolve_architecture",
]
