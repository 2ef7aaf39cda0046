"""One block: how a mixer, a feed-forward and their norms are arranged.

The arrangement is chosen by name per layer.  Built in:

``pre_norm``: x = norm(h); h += mixer(x); x = norm(h); h += ffn(x)
(prefixserve/model/llama.py:112-121, the only one that architecture uses).
``parallel``: both sublayers read the same stream, h += mixer(norm_a(h)) + ffn(norm_b(h)).

The residual stream h is float32.  A block takes and returns (h, pending):
``pending`` is a sublayer output that has not been added yet, because the sum
is done inside the next norm's kernel.  An arrangement is a function
``(block, h, pending, ctx, cache) -> (h, pending)`` over the block's parts
(``mixer_norm``, ``mixer``, ``ffn_norm``, ``ffn``; the last two are None in a
layer without feed-forward) and is added with ``register_arrangement``.
"""

from __future__ import annotations

from typing import Callable

from .. import ops
from ..config.spec import LayerSpec
from .base import CacheView, StepContext
from .registry import make

_ARRANGEMENTS: dict[str, Callable] = {}


def register_arrangement(name: str, run: Callable, *, replace: bool = False) -> None:
    if name in _ARRANGEMENTS and not replace:
        raise ValueError(f"block arrangement {name!r} is already registered")
    _ARRANGEMENTS[name] = run


class Block:
    def __init__(self, spec: LayerSpec):
        try:
            self.run = _ARRANGEMENTS[spec.arrangement]
        except KeyError:
            raise ValueError(f"block arrangement {spec.arrangement!r} is not registered (known: {sorted(_ARRANGEMENTS)})") from None
        self.mixer_norm = make("norm", spec.mixer_norm)
        self.mixer = make("mixer", spec.mixer)
        self.ffn_norm = make("norm", spec.ffn_norm) if spec.ffn_norm is not None else None
        self.ffn = make("ffn", spec.ffn) if spec.ffn is not None else None

    def named_parts(self):
        parts = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer)]
        if self.ffn is not None:
            parts += [("ffn_norm", self.ffn_norm), ("ffn", self.ffn)]
        return tuple(parts)

    def forward(self, h, pending, ctx: StepContext, cache: CacheView):
        return self.run(self, h, pending, ctx, cache)


def _sublayer(norm, part, h, pending, ctx, *more):
    """(stream after adding ``pending``, the part's output).  A part that takes a deferred input may have the sum
    and the norm done inside its first product, which then writes the summed stream to a new tensor."""
    if part.takes_deferred_input:
        x = norm.defer(h, pending, ctx)
        out = part.forward(x, ctx, *more)
        return x.residual(), out
    return h, part.forward(norm.forward(h, pending, ctx), ctx, *more)


def pre_norm(block: Block, h, pending, ctx: StepContext, cache: CacheView):
    h, pending = _sublayer(block.mixer_norm, block.mixer, h, pending, ctx, cache)
    if block.ffn is not None:
        h, pending = _sublayer(block.ffn_norm, block.ffn, h, pending, ctx)
    return h, pending


def parallel(block: Block, h, pending, ctx: StepContext, cache: CacheView):
    """Both sublayers see the stream as it entered the block (after ``pending``); their outputs are added together."""
    x = block.mixer_norm.forward(h, pending, ctx)       # h now holds the sum
    mixed = block.mixer.forward(x, ctx, cache)
    if block.ffn is None:
        return h, mixed
    fed = block.ffn.forward(block.ffn_norm.forward(h, None, ctx), ctx)
    ops.residual_add(h, mixed)
    return h, fed


register_arrangement("pre_norm", pre_norm)
register_arrangement("parallel", parallel)
