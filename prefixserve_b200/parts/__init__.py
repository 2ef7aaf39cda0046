from . import attention, embedding, ffn, norm, position  # noqa: F401  (registers the built-in kinds)
from .base import (CacheNeed, CacheView, FeedForward, FixedState, ItemView, Mixer, Norm, PagedKV, ParamSpec, Part,
                   PositionEncoding, StepContext)
from .block import Block, register_arrangement
from .model import DecoderModel, build_model
from .registry import (kinds, make, register_embedding, register_ffn, register_head, register_mixer, register_norm,
                       register_position)

__all__ = [
    "Block", "CacheNeed", "CacheView", "DecoderModel", "FeedForward", "FixedState", "ItemView", "Mixer", "Norm",
    "PagedKV", "ParamSpec", "Part", "PositionEncoding", "StepContext", "build_model", "kinds", "make",
    "register_arrangement", "register_embedding", "register_ffn", "register_head", "register_mixer", "register_norm", "register_position",
]
