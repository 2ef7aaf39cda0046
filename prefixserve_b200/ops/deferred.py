"""A normalised input that is computed by whoever consumes it.

A norm in front of a matrix product can hand over ``NormedRows`` instead of a
tensor.  ``ops.linear`` and ``ops.gated_linear`` then fold the residual sum and
the RMSNorm (prefixserve/model/llama.py:63-69, :117-121 of PrefixServe) into the
product's kernel where that kernel exists (few bfloat16 rows: the streaming
product keeps its share of the normalised row in registers) and otherwise ask
for the tensor, which runs the norm's own kernel once.  Either way the consumer
sees the same mathematics; ``residual()`` gives the float32 stream after the sum.
"""

from __future__ import annotations

import torch


class NormedRows:
    def __init__(self, h: torch.Tensor, pending: torch.Tensor | None, gain: torch.Tensor, eps: float,
                 dtype: torch.dtype, rows: torch.Tensor | None = None):
        self.h, self.pending, self.gain, self.eps, self.dtype, self.rows = h, pending, gain, float(eps), dtype, rows
        self._x: torch.Tensor | None = None
        self._settled = False      # the stream already holds h + pending
        self.shape = (h.shape[0] if rows is None else rows.numel(), h.shape[1])

    @classmethod
    def ready(cls, x: torch.Tensor, h: torch.Tensor) -> "NormedRows":
        """Wraps a row that a norm without a deferred form has already computed (h already updated)."""
        self = cls.__new__(cls)
        self.h, self.pending, self.gain, self.eps, self.dtype, self.rows = h, None, None, 0.0, x.dtype, None
        self._x, self._settled, self.shape = x, True, tuple(x.shape)
        return self

    @property
    def fusable(self) -> bool:
        return self._x is None and not self._settled

    def tensor(self) -> torch.Tensor:
        """The normalised rows as a tensor (computed once; adds ``pending`` into the stream in place unless ``rows``)."""
        if self._x is None:
            from .kernels import add_rmsnorm
            pending = None if self._settled else self.pending
            self._x = add_rmsnorm(self.h, pending, self.gain, self.eps, self.dtype, self.rows)
            self._settled = True
        return self._x

    def fused(self, new_h: torch.Tensor | None) -> None:
        """Told by a product that did the sum and the norm itself; ``new_h`` is the stream it wrote, if it wrote one."""
        if new_h is not None:
            self.h = new_h
        self._settled = True

    def residual(self) -> torch.Tensor:
        """The stream after the sum.  If nobody consumed the rows, the sum is done now."""
        if not self._settled:
            if self.rows is not None:
                raise RuntimeError("a row selection cannot update the residual stream")
            self.tensor()
        return self.h
