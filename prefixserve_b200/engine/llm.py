"""Python entry point: token ids in, token ids out.

    llm = LLM(model="folder", dtype="bfloat16")
    outputs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(max_tokens=8))

It is the reference's driver loop (schedule_step -> engine.step -> commit,
README.md:323-335 of PrefixServe, prefixserve/server.py:209-253) around this
engine and scheduler.
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from ..sampling import SamplingParams
from .engine import Engine, EngineConfig
from .loading import parse_dtype
from .scheduler import AddResult, Scheduler, SchedulerStats


class LLM:
    def __init__(self, model: str | Path, *, dtype: str | torch.dtype = "bfloat16", max_seq_len: int | None = None,
                 num_blocks: int | None = None, max_running_requests: int = 64, chunked_prefill_size: int = 512,
                 enable_prefix_cache: bool = True, max_waiting: int = 1024, page_size: int = 16,
                 device: str = "cuda", warm_up: bool = True, cast_float32_weights: bool = False) -> None:
        self.engine = Engine(EngineConfig(
            model_path=Path(model), dtype=parse_dtype(dtype), device=device, max_num_seqs=max_running_requests,
            max_prefill_tokens=chunked_prefill_size, max_seq_len=max_seq_len, num_blocks=num_blocks,
            page_size=page_size, enable_prefix_cache=enable_prefix_cache, cast_float32_weights=cast_float32_weights))
        self.scheduler = Scheduler(self.engine.cache, max_waiting=max_waiting, chunk_size=chunked_prefill_size,
                                   stop_token_ids=self.engine.stop_token_ids, enable_prefix_cache=enable_prefix_cache)
        self.max_running_requests = max_running_requests
        self.chunked_prefill_size = chunked_prefill_size
        self._counter = 0
        if warm_up:  # capture the decode step for every batch size up front instead of at its first use
            self.engine.capture_decode_graphs(range(1, max_running_requests + 1))

    def generate(self, prompts: Sequence[Sequence[int]], sampling: SamplingParams | Sequence[SamplingParams] | None = None
                 ) -> list[list[int]]:
        """Generates for every prompt (lists of token ids); returns the generated ids, in the order given."""
        if sampling is None:
            sampling = SamplingParams()
        per_prompt = list(sampling) if not isinstance(sampling, SamplingParams) else [sampling] * len(prompts)
        if len(per_prompt) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = []
        for prompt, sp in zip(prompts, per_prompt):
            rid = f"gen-{self._counter}"
            self._counter += 1
            verdict = self.scheduler.add_request(rid, list(prompt), sp.max_tokens, ignore_eos=sp.ignore_eos, sampling=sp)
            if verdict is not AddResult.ACCEPTED:
                for done in ids:
                    self.scheduler.free_request(done)
                raise ValueError(f"prompt {len(ids)} was refused: {verdict.value}")
            ids.append(rid)
        outputs: dict[str, list[int]] = {rid: [] for rid in ids}
        sched, engine = self.scheduler, self.engine
        pending = None  # the step on the device whose tokens have not been read yet
        try:
            while pending is not None or sched.has_work():
                if pending is None:
                    pending = engine.launch(sched.schedule_step(self.chunked_prefill_size, self.max_running_requests))
                # while that step runs: decide and launch the one after it, if that can be done without its tokens
                ahead = sched.schedule_ahead(self.max_running_requests)
                following = engine.launch(ahead, feed=pending) if ahead is not None else None
                result = sched.commit(pending.batch, engine.finish(pending))
                for rid, tok in result.new_tokens.items():
                    outputs[rid].append(tok)
                pending = following
            engine.check_device_status()
        except BaseException:
            # nothing of this call may outlive it: the batch in flight is forgotten, every request of the call is
            # ended and its slot and pages are given back, so that the next call starts clean
            sched.abandon_inflight()
            for rid in ids:
                sched.free_request(rid)
            raise
        return [outputs[rid] for rid in ids]

    def stats(self) -> SchedulerStats:
        return self.scheduler.stats()
