"""A single-GPU Llama inference engine for NVIDIA B200 (sm_100a)."""

from . import architectures  # noqa: F401  (registers LlamaForCausalLM)
from .config import LlamaConfig, Llama3RopeScaling, UnsupportedModelError, read_model_folder

from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["LLM", "Engine", "EngineConfig", "LlamaConfig", "Llama3RopeScaling", "SamplingParams", "Scheduler",
           "UnsupportedModelError", "read_model_folder"]


def __getattr__(name):  # the engine pulls in torch.cuda; load it only when asked for
    if name in ("LLM", "Engine", "EngineConfig", "Scheduler"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
