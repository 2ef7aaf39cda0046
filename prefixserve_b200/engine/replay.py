"""Trace replay: feeds given token ids through the model step by step and
writes logits.  It samples nothing and has no forward pass, cache or loader of
its own: it drives the same model, step function, cache manager and kernels
that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the offsets among them whose
logits are wanted; all entries of a step form one batch.  ``end``: requests
finished after this step; their pages and slot are given back.  When a step
wants anything, ``DIR/<step>.f32`` receives the logits as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After
every step the line ``done <step>`` is printed and flushed.

The cache pool is made for ``--max-tokens`` tokens (page granularity), so
pages are reused as requests end.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

from ..cache.manager import CacheManager, pages_for
from ..ops import library
from .loading import load_model, parse_dtype
from .step import EngineError, ModelRunner, StepItem

PAGE_SIZE = 16
LIVE_REQUESTS = 16  # slots; traces keep at most a handful of requests live


class Replayer:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, device: str = "cuda") -> None:
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device: trace replay runs the engine's kernels and has no CPU path")
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        _, _, self.model = load_model(model_dir, dtype=self.dtype, device=self.device)
        spec = self.model.spec
        pages = max(1, pages_for(max_tokens, PAGE_SIZE))
        max_seq_len = min(spec.max_positions, pages * PAGE_SIZE)
        self.cache = CacheManager(self.model.cache_needs(), num_pages=pages, num_slots=LIVE_REQUESTS,
                                  max_seq_len=max_seq_len, page_size=PAGE_SIZE, dtype=self.dtype, device=self.device,
                                  enable_prefix_cache=False)
        self.runner = ModelRunner(self.model, self.cache, device=self.device)
        self.slot_of: dict[str, int] = {}

    def run_step(self, record: dict) -> np.ndarray | None:
        """Runs one step of the trace; returns float32 [wanted, vocab] or None when nothing was wanted."""
        items: list[StepItem] = []
        for entry in record.get("entries", []):
            rid = str(entry["id"])
            tokens = np.asarray(entry["tokens"], dtype=np.int32)
            if rid not in self.slot_of:
                slot = self.cache.open()
                if slot is None:
                    raise EngineError(f"request {rid!r}: more than {LIVE_REQUESTS} requests are live")
                self.slot_of[rid] = slot
            slot = self.slot_of[rid]
            start = self.cache.position(slot)
            if not self.cache.reserve(slot, start + len(tokens)):
                raise EngineError(f"request {rid!r}: the pool of {self.cache.num_pages(0)} pages (--max-tokens) is exhausted")
            items.append(StepItem(slot, start, tokens, tuple(int(w) for w in entry.get("want", []))))
        logits = self.runner.step(items) if items else None
        for it in items:
            self.cache.advance(it.slot, it.start + len(it.tokens))
        out = None
        if logits is not None and logits.shape[0] > 0:
            out = logits.to("cpu").numpy().astype("<f4", copy=False)
            if self.dtype == torch.bfloat16:  # the device has just been waited for: see whether a bounded wait gave up
                status = library.tcgen05_status()
                if status:
                    raise EngineError(f"a tcgen05 kernel gave up waiting on a barrier (status {status:#x}); results are void")
        for rid in record.get("end", []):
            slot = self.slot_of.pop(str(rid), None)
            if slot is not None:
                self.cache.close(slot)
        return out


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine, write logits")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    args = p.parse_args(argv)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    replayer = Replayer(args.model, args.dtype, args.max_tokens)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = replayer.run_step(record)
        if logits is not None:
            logits.tofile(out_dir / f"{step}.f32")
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
