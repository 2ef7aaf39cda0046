"""Runs the sampling kernel for the rows of a step."""

from __future__ import annotations

from typing import Sequence

import torch

from .. import ops
from . import SamplingParams


def choose_tokens(logits: torch.Tensor, params: Sequence[SamplingParams], positions: Sequence[int]) -> torch.Tensor:
    """logits float32 [S, V] on the device -> int32 [S] on the device.

    ``positions[i]`` is the absolute position of the token being chosen for row i.
    """
    if all(p.temperature == 0 for p in params):
        return ops.sample(logits)
    dev = logits.device
    temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=dev)
    seed = torch.tensor([p.seed for p in params], dtype=torch.int64, device=dev)
    position = torch.tensor(list(positions), dtype=torch.int32, device=dev)
    return ops.sample(logits, temperature, seed, position)
