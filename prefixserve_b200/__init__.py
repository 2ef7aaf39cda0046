"""A single-GPU Llama inference engine for NVIDIA B200 (sm_100a)."""

from . import architectures  # noqa: F401  (registers LlamaForCausalLM)
from .config import LlamaConfig, Llama3RopeScaling, UnsupportedModelError, read_model_folder

__version__ = "0.1.0"
__all__ = ["LlamaConfig", "Llama3RopeScaling", "UnsupportedModelError", "read_model_folder"]
