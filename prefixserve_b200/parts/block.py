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
        x = self.mixer_norm.forward(h, pending, ctx)
        pending = self.mixer.forward(x, ctx, cache)
        x = self.ffn_norm.forward(h, pending, ctx)
        pending = self.ffn.forward(x, ctx)
        return h, pending
