"""Gated feed-forward: down(act(gate(x)) * up(x)), gate and up fused into one
matrix (prefixserve/model/llama.py:120-121, prefixserve/model/weights.py:120-123)."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, ParamSpec, StepContext
from .registry import register_ffn


class GatedMLP(FeedForward):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_deferred_input = True  # x goes to one product only, which may do the norm in front of it itself

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not built (one of {sorted(ops.ACTIVATIONS)})")
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def param_specs(self):
        return {
            "gate_proj": ParamSpec((self.inter, self.hidden)),
            "up_proj": ParamSpec((self.inter, self.hidden)),
            "down_proj": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors, *, compute_dtype, device):
        g, u = tensors["gate_proj"], tensors["up_proj"]
        dtype = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dtype), u.to(dtype)], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def forward(self, x, ctx: StepContext):
        return ops.last_product(ops.gated_linear(x, self.w_gate_up, self.activation), self.w_down, ctx)


register_ffn("gated_mlp", GatedMLP, replace=True)
