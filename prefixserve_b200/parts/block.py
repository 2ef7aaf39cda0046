"""One block: how a mixer, a feed-forward and their norms are arranged.

``pre_norm``: x = norm(h); h += mixer(x); x = norm(h); h += ffn(x)
(prefixserve/model/llama.py:112-121).  The residual stream h is float32; the
sum with a sublayer's output is done inside the next norm's kernel, so a block
takes and returns (h, pending output).
"""

from __future__ import annotations

from ..config.spec import LayerSpec
from .base import CacheView, StepContext
from .registry import make


class Block:
    def __init__(self, spec: LayerSpec):
        if spec.arrangement != "pre_norm":
            raise ValueError(f"block arrangement {spec.arrangement!r} is not built (only pre_norm)")
        self.mixer_norm = make("norm", spec.mixer_norm)
        self.mixer = make("mixer", spec.mixer)
        self.ffn_norm = make("norm", spec.ffn_norm)
        self.ffn = make("ffn", spec.ffn)

    def named_parts(self):
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer), ("ffn_norm", self.ffn_norm), ("ffn", self.ffn))

    def forward(self, h, pending, ctx: StepContext, cache: CacheView):
        h, pending = _sublayer(self.mixer_norm, self.mixer, h, pending, ctx, cache)
        h, pending = _sublayer(self.ffn_norm, self.ffn, h, pending, ctx)
        return h, pending


def _sublayer(norm, part, h, pending, ctx, *more):
    """(stream after adding ``pending``, the part's output).  A part that takes a deferred input may have the sum
    and the norm done inside its first product, which then writes the summed stream to a new tensor."""
    if part.takes_deferred_input:
        x = norm.defer(h, pending, ctx)
        out = part.forward(x, ctx, *more)
        return x.residual(), out
    return h, part.forward(norm.forward(h, pending, ctx), ctx, *more)
