"""Reads a model folder's safetensors by tensor name and hands each part its tensors.

Files: ``model.safetensors.index.json`` (its shard list) or a single
``model.safetensors`` (prefixserve/model/weights.py:62-70).  Every wanted
tensor is looked up by the checkpoint name the architecture gives for its part
path and its shape is compared before anything is read; all problems (missing,
unexpected, wrong shape) are reported together in one ``WeightLoadError``.

Stored types are kept: 16-bit matrices stay bfloat16 on the bfloat16 path, a
tensor stored in 32-bit stays float32 (the products then take the float32
kernel), gains are widened to float32 (exact), integer tables become int32.
On the float32 path everything is widened to float32.  With
``cast_float32=True`` matrices stored in 32-bit are rounded to the compute
type at load instead, which is what the reference does with every tensor
(prefixserve/model/weights.py:94-98): a float32 checkpoint then runs on the
tensor cores like a bfloat16 one.
"""

from __future__ import annotations

import json
import sys
from contextlib import ExitStack
from pathlib import Path
from typing import Callable, Mapping

import torch
from safetensors import safe_open

from ..parts.base import ParamSpec


class WeightLoadError(RuntimeError):
    pass


_INT_TYPES = {torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool}
_STR_TO_DTYPE = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
                 "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
                 "BOOL": torch.bool}


def shard_files(folder: Path) -> list[Path]:
    index = folder / "model.safetensors.index.json"
    if index.exists():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [folder / n for n in names]
    single = folder / "model.safetensors"
    if single.exists():
        return [single]
    raise WeightLoadError(f"{folder} holds neither model.safetensors nor model.safetensors.index.json")


def held_dtype(role: str, stored: torch.dtype, compute_dtype: torch.dtype, cast_float32: bool = False) -> torch.dtype:
    """The type a tensor has on the device, from its role, its stored type and the path's compute type."""
    if role == "table_int" or stored in _INT_TYPES:
        return torch.int32
    if compute_dtype == torch.float32 or role == "vector":
        return torch.float32
    if stored in (torch.float32, torch.float64) and not cast_float32:
        return torch.float32  # stored in 32-bit: stays so
    return compute_dtype


def load_tensors(
    folder: str | Path,
    wanted: Mapping[str, ParamSpec],
    tensor_name: Callable[[str], str],
    ignorable: Callable[[str], bool],
    *,
    compute_dtype: torch.dtype,
    device: torch.device | str,
    cast_float32: bool = False,
) -> dict[str, torch.Tensor]:
    """part path -> tensor on ``device``.  Raises one WeightLoadError naming every problem."""
    folder = Path(folder)
    device = torch.device(device)
    files = shard_files(folder)
    absent = [f for f in files if not f.exists()]
    if absent:
        raise WeightLoadError(f"shards named by the index are missing: {[f.name for f in absent]}")
    with ExitStack() as stack:
        where: dict[str, object] = {}
        for f in files:
            handle = stack.enter_context(safe_open(str(f), framework="pt", device="cpu"))
            for name in handle.keys():
                where[name] = handle

        names = {path: tensor_name(path) for path in wanted}
        missing, misshapen = [], []
        for path, spec in wanted.items():
            name = names[path]
            handle = where.get(name)
            if handle is None:
                missing.append(name)
                continue
            got = tuple(handle.get_slice(name).get_shape())
            if got != tuple(spec.shape):
                misshapen.append(f"{name}: file has {got}, model wants {tuple(spec.shape)}")
        used = set(names.values())
        unexpected = sorted(n for n in where if n not in used and not ignorable(n))
        if missing or misshapen or unexpected:
            lines = [f"cannot load weights from {folder}:"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
            if misshapen:
                lines.append(f"  wrong shape ({len(misshapen)}): " + "; ".join(misshapen))
            raise WeightLoadError("\n".join(lines))

        out: dict[str, torch.Tensor] = {}
        wide = 0
        for path, spec in wanted.items():
            t: torch.Tensor = where[names[path]].get_tensor(names[path])  # type: ignore[attr-defined]
            out[path] = t.to(device=device, dtype=held_dtype(spec.role, t.dtype, compute_dtype, cast_float32)).contiguous()
            wide += spec.role != "vector" and t.dim() >= 2 and out[path].dtype == torch.float32 and compute_dtype != torch.float32
        if wide:  # right, but not what somebody who asked for bfloat16 may expect of the speed
            print(f"[prefixserve_b200] {wide} matrices of {folder} are stored in 32-bit and stay so: their products run on the "
                  f"float32 kernel, not on the tensor cores (cast_float32_weights / --cast-float32-weights rounds them at "
                  f"load instead)", file=sys.stderr, flush=True)
        return out


def convert_tensors(tensors: Mapping[str, torch.Tensor], wanted: Mapping[str, ParamSpec], *,
                    compute_dtype: torch.dtype, device: torch.device | str) -> dict[str, torch.Tensor]:
    """Same placement rules for tensors that are already in memory (random weights without a folder)."""
    problems = []
    for path, spec in wanted.items():
        if path not in tensors:
            problems.append(f"missing {path}")
        elif tuple(tensors[path].shape) != tuple(spec.shape):
            problems.append(f"{path}: has {tuple(tensors[path].shape)}, model wants {tuple(spec.shape)}")
    extra = sorted(set(tensors) - set(wanted))
    if extra:
        problems.append("unexpected " + ", ".join(extra))
    if problems:
        raise WeightLoadError("cannot use the given tensors: " + "; ".join(problems))
    return {
        path: tensors[path].to(device=device, dtype=held_dtype(spec.role, tensors[path].dtype, compute_dtype)).contiguous()
        for path, spec in wanted.items()
    }
