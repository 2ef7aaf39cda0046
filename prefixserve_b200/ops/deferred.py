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


class PendingProduct:
    """A sublayer's last product, x @ w^T, that has not run yet.  Its only reader is the residual sum in front of the
    next norm, and for a few dozen rows that sum, the gain and the sums of squares ride in the product's own epilogue
    (``NormedRows.raw``); everybody else asks for ``tensor()``, which runs the product as usual."""

    def __init__(self, x: torch.Tensor, w: torch.Tensor):
        self.x, self.w = x, w
        self.shape, self.dtype = (x.shape[0], w.shape[0]), x.dtype
        self._y: torch.Tensor | None = None

    def tensor(self) -> torch.Tensor:
        if self._y is None:
            from .kernels import linear
            self._y = linear(self.x, self.w)
        return self._y


class NormedRows:
    def __init__(self, h: torch.Tensor, pending, gain: torch.Tensor, eps: float,
                 dtype: torch.dtype, rows: torch.Tensor | None = None):
        if rows is not None and isinstance(pending, PendingProduct):
            pending = pending.tensor()
        self.h, self.pending, self.gain, self.eps, self.dtype, self.rows = h, pending, gain, float(eps), dtype, rows
        self._raw = None           # (gained rows, shares of the sums of squares) once the product in front has left them
        self._x: torch.Tensor | None = None
        self._settled = False      # the stream already holds h + pending
        self.shape = (h.shape[0] if rows is None else rows.numel(), h.shape[1])

    @classmethod
    def ready(cls, x: torch.Tensor, h: torch.Tensor) -> "NormedRows":
        """Wraps a row that a norm without a deferred form has already computed (h already updated)."""
        self = cls.__new__(cls)
        self.h, self.pending, self.gain, self.eps, self.dtype, self.rows = h, None, None, 0.0, x.dtype, None
        self._x, self._settled, self.shape, self._raw = x, True, tuple(x.shape), None
        return self

    @property
    def fusable(self) -> bool:
        return self._x is None and not self._settled and not isinstance(self.pending, PendingProduct)

    def raw(self):
        """(v * gain as bfloat16 [M, K], the tiles' shares of every row's sum(v^2) float32 [parts, 64]) with v = h + pending,
        or None.  Only when ``pending`` is a product that has not run: it runs now, on the few-row kernel, with the
        residual sum in its epilogue (the stream is updated in place).  The consumer multiplies the gained rows by its
        weights and scales the sums by rsqrt(sum(v^2) / K + eps)."""
        if self._raw is None and isinstance(self.pending, PendingProduct) and not self._settled and self.rows is None:
            from .tensorcore import fewrows_add_norm
            self._raw = fewrows_add_norm(self.pending.x, self.pending.w, self.h, self.gain)
            if self._raw is not None:
                self._settled = True
        return self._raw

    def tensor(self) -> torch.Tensor:
        """The normalised rows as a tensor (computed once; adds ``pending`` into the stream in place unless ``rows``)."""
        if self._x is None:
            from .kernels import add_rmsnorm
            pending = None if self._settled else self.pending
            if isinstance(pending, PendingProduct):
                pending = pending.tensor()
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
