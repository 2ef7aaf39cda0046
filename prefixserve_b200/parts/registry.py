"""Registries of part kinds.  A configuration names parts by kind; tests and
other architectures add kinds with the ``register_*`` functions and need no
change to the engine."""

from __future__ import annotations

from typing import Any, Callable, Mapping

from ..config.spec import PartSpec

_KINDS: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str, factory: Callable[..., Any], replace: bool) -> None:
    table = _KINDS[family]
    if kind in table and not replace:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    table[kind] = factory


def register_mixer(kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    _register("mixer", kind, factory, replace)


def register_ffn(kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    _register("ffn", kind, factory, replace)


def register_norm(kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    _register("norm", kind, factory, replace)


def register_position(kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    _register("position", kind, factory, replace)


def register_embedding(kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    _register("embedding", kind, factory, replace)


def register_head(kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    _register("head", kind, factory, replace)


def make(family: str, spec: PartSpec | Mapping[str, Any]) -> Any:
    if not isinstance(spec, PartSpec):
        spec = PartSpec(str(spec["kind"]), {k: v for k, v in spec.items() if k != "kind"})
    table = _KINDS[family]
    if spec.kind not in table:
        raise KeyError(f"no {family} of kind {spec.kind!r}; registered: {sorted(table)}")
    return table[spec.kind](spec.params)


def kinds(family: str) -> list[str]:
    return sorted(_KINDS[family])
