"""Position encodings.

``rope``: rotary angles per (position, pair), float32 tables built once at
start-up with the formulas of prefixserve/model/llama.py:24-60: inverse
frequencies 1/theta^(2j/D); with llama3 scaling, wavelengths longer than
original/low_freq_factor are divided by ``factor``, those shorter than
original/high_freq_factor are kept, and the band between is blended.  The
tables hold D/2 columns (the reference's table repeats them to D).
``none``: no rotation; queries and keys go through unchanged.

What a rotating part tells its mixer: ``cos``/``sin`` float32 [positions,
rotary_dim/2], ``rotary_dim`` (how many leading elements of a head turn;
default all) and ``layout`` ("half": element j turns with j + rotary_dim/2;
"interleaved": 2j with 2j+1).  The attention part hands that description to
its kernels; those that bake in the split-half rotation of a whole head are
only used when the description says exactly that.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_position


def rope_inverse_frequencies(head_dim: int, theta: float, scaling) -> torch.Tensor:
    exponents = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
    inv = 1.0 / (theta ** exponents)
    if not scaling:
        return inv
    kind = scaling.get("kind")
    if kind != "llama3":
        raise ValueError(f"rope scaling kind {kind!r} is not built")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = float(scaling["original_max_positions"])
    wavelength = 2 * math.pi / inv
    long_limit, short_limit = original / low, original / high
    stretched = torch.where(wavelength > long_limit, inv / factor, inv)
    blend = (original / wavelength - low) / (high - low)
    blended = (1 - blend) * stretched / factor + blend * stretched
    in_band = (~(wavelength < short_limit)) & (~(wavelength > long_limit))
    return torch.where(in_band, blended, stretched)


_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


class RotaryEncoding(PositionEncoding):
    rotates = True

    def __init__(self, params):
        super().__init__(params)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        self.scaling = params.get("scaling")
        self.layout = str(params.get("layout", "half"))
        if self.layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout {self.layout!r} is not built (half or interleaved)")
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or not 2 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within the head size {self.head_dim}")
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None

    def prepare(self, *, max_positions, compute_dtype, device):
        # layers with the same constants share one pair of tables
        key = (self.rotary_dim, self.theta, repr(sorted(self.scaling.items())) if self.scaling else None, str(device))
        held = _TABLES.get(key)
        if held is None or held[0].shape[0] < max_positions:
            inv = rope_inverse_frequencies(self.rotary_dim, self.theta, self.scaling)
            angles = torch.outer(torch.arange(max_positions, dtype=torch.int64).float(), inv)  # float32, on the host
            held = (angles.cos().to(device).contiguous(), angles.sin().to(device).contiguous())
            _TABLES[key] = held
        self.cos, self.sin = held


class NoPositions(PositionEncoding):
    rotates = False
    cos = None
    sin = None
    rotary_dim = None
    layout = "half"


register_position("rope", RotaryEncoding, replace=True)
register_position("none", NoPositions, replace=True)
