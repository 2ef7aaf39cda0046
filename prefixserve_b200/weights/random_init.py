"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode (its tests build random models through another
library, tests/test_llama_exact.py:82-85).  Tensors are drawn on the host with
one seeded generator, in the order of the model's parameter table, so the same
(configuration, seed) always gives the same file: matrices N(0, std), gains 1
or 1 + N(0, gain_noise).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch
from safetensors.torch import save_file

from ..config.registry import get_architecture
from ..parts.base import ParamSpec
from ..parts.model import build_model


def random_tensors(table: Mapping[str, ParamSpec], seed: int, *, std: float = 0.02, gain_noise: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16, device: str = "cpu") -> dict[str, torch.Tensor]:
    """part path -> tensor (on the host), drawn in table order from one generator.  ``device``: where the numbers
    are drawn; the host's generator and a GPU's give different (each reproducible) values, so tests that compare
    with stored outputs draw on the host, and benchmarks of billions of weights may draw on the GPU."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for path, spec in table.items():
        if spec.role == "table_int":
            out[path] = torch.zeros(spec.shape, dtype=torch.int32)
        elif spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if gain_noise:
                t += gain_noise * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
            out[path] = t.to(dtype).cpu()
        else:
            out[path] = (std * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)).to(dtype).cpu()
    return out


def write_random_model(folder: str | Path, config: Any, seed: int, *, std: float = 0.02, gain_noise: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16, architecture: str | None = None, device: str = "cpu") -> Path:
    """Writes config.json and model.safetensors for ``config`` (a typed configuration with ``to_config_json``)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = get_architecture(architecture or config.architecture)
    model = build_model(arch.to_spec(config))
    table = model.param_table()
    by_path = random_tensors(table, seed, std=std, gain_noise=gain_noise, dtype=dtype, device=device)
    by_name = {arch.tensor_name(path): t.contiguous() for path, t in by_path.items()}
    save_file(by_name, str(folder / "model.safetensors"), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config.to_config_json(), indent=2) + "\n")
    return folder
