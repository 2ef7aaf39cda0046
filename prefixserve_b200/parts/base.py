"""What every part of a model has in common, and what a part sees of a step.

A part is built from a ``PartSpec`` (its kind plus sizes and constants),
declares the tensors it needs by local name, receives them once, and then runs
on the tokens of a step.  It never learns which model it sits in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part wants from the checkpoint.

    role: "matrix" (operand of a matrix product: held in the compute dtype
    unless the file stores it in 32-bit), "vector" (norm gains and the like:
    always widened to float32, which is exact), or "table_int" (int32).
    init: how the random-weights mode fills it ("normal" or "ones").
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKV:
    """Keys and values for every token (or the last ``window`` of them)."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    key_order: str = "natural"  # how a key head's elements are ordered in the pages; writer and readers must agree


@dataclass(frozen=True)
class FixedState:
    """A per-request tensor of fixed shape that a mixer carries across steps."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeed:
    paged: PagedKV | None = None
    state: FixedState | None = None


@dataclass
class CacheView:
    """The cache entry a mixer call works on."""

    group: int | None          # which page table of the step applies (None: no pages)
    kv: torch.Tensor | None    # [num_pages, 2, num_kv_heads, page_size, head_dim]
    state: torch.Tensor | None  # [num_slots, *shape]
    page_size: int
    writes: bool = True


@dataclass(frozen=True)
class ItemView:
    """Host-side view of one batch item: tokens [start, end) of one request."""

    slot: int
    start: int
    end: int
    first_token: int  # offset of its first token in the flat batch


@dataclass
class StepContext:
    """Everything about the current batch that parts may read."""

    num_tokens: int
    num_items: int
    compute_dtype: torch.dtype
    device: torch.device
    items: Sequence[ItemView]            # host side
    token_ids: torch.Tensor              # [T] int32
    positions: torch.Tensor              # [T] int32, absolute
    token_item: torch.Tensor             # [T] int32, index into items
    item_start: torch.Tensor             # [B+1] int32, offsets into the flat batch
    kv_len: torch.Tensor                 # [B] int32, tokens held after this step
    slots: torch.Tensor                  # [B] int32
    block_tables: Mapping[int, torch.Tensor]   # group -> [B, width] int32, by absolute page index
    max_new_tokens: int                  # longest item of the step
    max_kv_len: int                      # largest kv_len of the step
    all_decode: bool                     # every item brings exactly one token
    extras: dict[str, Any] = field(default_factory=dict)


class Part:
    """Base class; subclasses override what they need."""

    # A mixer, feed-forward or head that hands its input straight to ``ops.linear`` / ``ops.gated_linear`` sets this
    # and then receives an ``ops.NormedRows`` instead of a tensor (see ``Norm.defer``).
    takes_deferred_input = False

    # True when forward() launches the same device work for the same tensor shapes, reading everything that varies
    # from device memory (then a decode step can be captured once and replayed).  A part that loops over
    # ``ctx.items`` on the host must leave this False.
    graph_safe = False

    def __init__(self, spec_params: Mapping[str, Any]) -> None:
        self.params = dict(spec_params)

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], *, compute_dtype: torch.dtype, device: torch.device) -> None:
        """Receives the tensors named in param_specs (already on the device)."""

    def prepare(self, *, max_positions: int, compute_dtype: torch.dtype, device: torch.device) -> None:
        """Builds start-up tables that depend on engine limits (e.g. rotary angles)."""


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:  # [T,H] -> [T,H]
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, h: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """h: float32 residual stream [T,H]; delta: pending sublayer output or None.

        Adds delta into h (in place, in float32) and returns the normalised
        rows in the compute dtype.  With ``rows`` only those rows are read and
        h is left untouched (last use of the stream).
        """
        raise NotImplementedError

    def defer(self, h: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext, rows: torch.Tensor | None = None):
        """Same, for a consumer that declares ``takes_deferred_input``: returns an ``ops.NormedRows``, which the
        consumer passes to ``ops.linear`` / ``ops.gated_linear`` (they may do the norm inside the product) or turns
        into a tensor with ``.tensor()``.  A norm without a deferred form computes now and wraps the result."""
        from ..ops import NormedRows
        return NormedRows.ready(self.forward(h, delta, ctx, rows), h)


class PositionEncoding(Part):
    pass
