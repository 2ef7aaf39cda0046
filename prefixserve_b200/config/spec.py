"""Architecture-neutral description of a decoder: which parts, in which order.

A model is data: a tuple of layer descriptions (each naming a mixer, a
feed-forward and two norms by *kind* plus their sizes), and a run list that
says which layer runs when and which cache entry it uses.  The builder in
``prefixserve_b200.parts.model`` turns this into objects through the part
registries; nothing here knows about any particular architecture.

The reference hard-wires this structure inside one forward function
(prefixserve/model/llama.py:87-126); here it is a value so that another
architecture only has to produce another ``ModelSpec``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part, named by registry kind, with its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def with_params(self, **changes: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(changes)
        return PartSpec(self.kind, merged)


def part(kind: str, **params: Any) -> PartSpec:
    return PartSpec(kind, params)


@dataclass(frozen=True)
class LayerSpec:
    """One block: a mixer, a feed-forward and their norms, put together by the named arrangement
    (``parts.block``: "pre_norm", "parallel", or one registered there).  ``ffn`` and ``ffn_norm`` may be None: a
    layer that only mixes."""

    mixer: PartSpec
    ffn: PartSpec | None
    mixer_norm: PartSpec
    ffn_norm: PartSpec | None
    arrangement: str = "pre_norm"

    def __post_init__(self) -> None:
        if (self.ffn is None) != (self.ffn_norm is None):
            raise ValueError("a layer has a feed-forward and its norm, or neither")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run list.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may appear several times:
    shared weights).  ``cache`` names the cache entry the mixer uses; entries
    are numbered per model, and two calls naming the same entry share keys and
    values.  Only a call with ``writes_cache`` appends to its entry; a call
    that merely reads another call's entry must come after it in the list.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: frozenset[int] = frozenset()

    def __post_init__(self) -> None:
        problems = []
        owners: dict[int, int] = {}
        for i, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                problems.append(f"run list entry {i} names layer {call.layer}, model has {len(self.layers)}")
                continue
            if call.writes_cache:
                if call.cache in owners:
                    problems.append(f"cache entry {call.cache} is written by run list entries {owners[call.cache]} and {i}")
                owners[call.cache] = i
            elif call.cache not in owners:
                problems.append(f"run list entry {i} reads cache entry {call.cache} before anything wrote it")
        if problems:
            raise ValueError("bad model description: " + "; ".join(problems))

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((c.cache for c in self.schedule), default=-1)


def sequential_schedule(num_layers: int) -> tuple[LayerCall, ...]:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(LayerCall(layer=i, cache=i) for i in range(num_layers))
