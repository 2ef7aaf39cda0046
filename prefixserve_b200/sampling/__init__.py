"""How the next token is chosen.

The reference samples greedily only (torch.argmax,
prefixserve/llama_engine.py:146; its server refuses temperature > 0,
prefixserve/server.py:334-337).  Here temperature 0 is the same arg max and a
positive temperature draws from softmax(logits / temperature) with a
generator keyed by (seed, position), so a request's draws do not depend on the
batch it happens to run in.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0
    max_tokens: int = 16
    ignore_eos: bool = False
    stop_token_ids: tuple[int, ...] = ()   # this request also ends on these (beside the model's own stop ids)

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))


GREEDY = SamplingParams()

__all__ = ["GREEDY", "SamplingParams"]
