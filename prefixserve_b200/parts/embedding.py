"""Token embedding and LM head (prefixserve/model/llama.py:109, :125-126).

The embedding gathers rows straight into the float32 residual stream.  The
head multiplies the normalised, selected rows by [vocab, hidden]^T and returns
float32 logits; when tied it uses the embedding's tensor.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import ParamSpec, Part
from .registry import register_embedding, register_head


class TokenEmbedding(Part):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.table: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors, *, compute_dtype, device):
        self.table = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.table)


class LMHead(Part):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_deferred_input = True  # x goes to one product only, which may do the norm in front of it itself

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied = bool(params.get("tied", False))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors, *, compute_dtype, device):
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)


register_embedding("token_embedding", TokenEmbedding, replace=True)
register_head("lm_head", LMHead, replace=True)
