"""Model folder -> model with its weights on the device."""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from .. import architectures  # noqa: F401  (registers the shipped architectures)
from ..config.registry import Architecture, read_model_folder
from ..parts.model import DecoderModel, build_model
from ..weights.loader import load_tensors

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def parse_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in DTYPES.values():
            raise ValueError(f"dtype {name} is not built (bfloat16 or float32)")
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not built (bfloat16 or float32)") from None


def load_model(folder: str | Path, *, dtype: torch.dtype, device: torch.device | str,
               max_positions: int | None = None, cast_float32: bool = False) -> tuple[Architecture, Any, DecoderModel]:
    """Reads config.json, picks the model by its architecture name, loads the weights by tensor name."""
    arch, config = read_model_folder(folder)
    spec = arch.to_spec(config)
    model = build_model(spec)
    tensors = load_tensors(folder, model.param_table(), arch.tensor_name, lambda n: arch.ignorable(config, n),
                           compute_dtype=dtype, device=device, cast_float32=cast_float32)
    limit = spec.max_positions if max_positions is None else min(max_positions, spec.max_positions)
    model.load(tensors, compute_dtype=dtype, device=torch.device(device), max_positions=limit)
    return arch, config, model
