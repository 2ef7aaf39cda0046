"""Runs the sampling kernel for the rows of a step."""

from __future__ import annotations

import torch

from .. import ops


def choose_tokens(logits: torch.Tensor, records: torch.Tensor, row_slots: torch.Tensor) -> torch.Tensor:
    """logits float32 [S, V] on the device -> int32 [S] on the device.

    ``row_slots[i]`` is the request slot of row i; the row's temperature, seed and the absolute position of the
    token being chosen are read on the device from that slot's record (``CacheManager.records_dev``), where
    admission and the step itself have put them.  Nothing is built on the host for a step.
    """
    return ops.sample_slots(logits, records, row_slots)
