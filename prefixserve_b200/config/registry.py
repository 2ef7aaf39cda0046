"""One registry: architecture name (config.json ``architectures[0]``) -> model.

The reference only checks ``model_type == "llama"``
(prefixserve/model/config.py:64) and builds its one model directly; here the
name picks an ``Architecture`` record that knows how to read that
architecture's config.json, how to describe the model as parts, and how its
checkpoint names its tensors.  Adding an architecture is one ``register``
call; nothing else in the engine names a model.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .spec import ModelSpec


class UnknownArchitectureError(ValueError):
    pass


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: tuple[str, ...]
    read_config: Callable[[Mapping[str, Any], Mapping[str, Any] | None], Any]
    to_spec: Callable[[Any], ModelSpec]
    # part path ("layers.3.mixer.q_proj") -> tensor name in the checkpoint
    tensor_name: Callable[[str], str]
    # tensors a checkpoint may carry that the model never reads
    ignorable: Callable[[Any, str], bool] = lambda cfg, name: False


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitectureError(
            f"no model is registered for architecture {name!r}; registered: {registered_architectures()}"
        ) from None


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    """Picks the record from a parsed config.json."""
    names = raw.get("architectures") or []
    if names:
        return get_architecture(str(names[0]))
    # Hand-written folders sometimes give only model_type.
    mt = raw.get("model_type")
    for arch in _ARCHITECTURES.values():
        if mt in arch.model_types:
            return arch
    raise UnknownArchitectureError(
        f"config.json names no architecture (architectures={names!r}, model_type={mt!r}); "
        f"registered: {registered_architectures()}"
    )


def read_model_folder(folder: str | Path) -> tuple[Architecture, Any]:
    """config.json (+ generation_config.json) -> (architecture record, typed config)."""
    folder = Path(folder)
    cfg_file = folder / "config.json"
    if not cfg_file.exists():
        raise FileNotFoundError(f"{folder} has no config.json")
    raw = json.loads(cfg_file.read_text())
    gen_file = folder / "generation_config.json"
    gen = json.loads(gen_file.read_text()) if gen_file.exists() else None
    arch = architecture_of(raw)
    return arch, arch.read_config(raw, gen)
