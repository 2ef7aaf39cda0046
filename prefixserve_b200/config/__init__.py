from .llama import Llama3RopeScaling, LlamaConfig, UnsupportedModelError
from .registry import (
    Architecture,
    UnknownArchitectureError,
    architecture_of,
    get_architecture,
    read_model_folder,
    register_architecture,
    registered_architectures,
)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec, part, sequential_schedule

__all__ = [
    "Architecture", "LayerCall", "LayerSpec", "Llama3RopeScaling", "LlamaConfig", "ModelSpec", "PartSpec",
    "UnknownArchitectureError", "UnsupportedModelError", "architecture_of", "get_architecture", "part",
    "read_model_folder", "register_architecture", "registered_architectures", "sequential_schedule",
]
