"""RMSNorm, fused with the residual sum that precedes it.

y = gain * (x * rsqrt(mean(x^2) + eps)), everything in float32
(prefixserve/model/llama.py:63-69).  The residual stream is float32; the
pending output of the previous sublayer is added in the same kernel that
normalises (prefixserve/model/llama.py:117,:119,:121).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, ParamSpec, StepContext
from .registry import register_norm


class RMSNorm(Norm):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_pending_products = True  # ``delta`` may be an ops.PendingProduct (a product that has not run yet)

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.gain: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), role="vector", init="ones")}

    def load(self, tensors, *, compute_dtype, device):
        self.gain = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h, delta, ctx: StepContext, rows=None):
        return ops.add_rmsnorm(h, delta, self.gain, self.eps, ctx.compute_dtype, rows)

    def defer(self, h, delta, ctx: StepContext, rows=None):
        return ops.NormedRows(h, delta, self.gain, self.eps, ctx.compute_dtype, rows)


register_norm("rms", RMSNorm, replace=True)
