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
pages are reused as requests end.  ``--max-live`` (default 64) is the number of
request slots, ``--page-size`` (default 16) the tokens per page.

``--mode scheduler`` replays through the scheduler instead: the lines say when
requests arrive, the scheduler decides the batches (prefix hits, portions
under the token budget, preemption and recomputation, steps launched ahead,
captured decode steps), and every sampled token is replaced by the one the
trace gives, as the reference's tests do at commit
(tests/test_llama_exact.py:130-167, tests/gpu/test_engine_flashinfer.py:50-77
of PrefixServe):

    {"step": 0, "add": [{"id": "a", "prompt": [5, 17, 3], "forced": [9, 2, 4]}], "abort": []}

Each line is one scheduler step (``add`` and ``abort`` may be absent).  A
request generates ``len(forced)`` tokens.  ``DIR/<step>.f32`` holds the logits
of the step's sampling positions and ``DIR/<step>.json`` says which they are:
``{"rows": [{"id": "a", "position": 3}], "preempted": [...], "finished": {...}}``
where ``position`` is the index, in prompt + forced, of the token the row
predicts.  When the input ends, a line ``stats {...}`` with the scheduler's
and the engine's counters is printed.  Pool and limits: ``--max-tokens``
(pool), ``--max-seq-len``, ``--chunk`` (token budget and longest portion),
``--max-running``, ``--no-prefix-cache``, ``--no-ahead``, ``--no-graphs``.
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

PAGE_SIZE = 16       # default tokens per page
LIVE_REQUESTS = 64   # default number of request slots


class Replayer:
    """Step mode: the trace names every batch; this drives the step function on the real cache."""

    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, device: str = "cuda", *,
                 max_live: int = LIVE_REQUESTS, page_size: int = PAGE_SIZE, use_graphs: bool = True) -> None:
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device: trace replay runs the engine's kernels and has no CPU path")
        if max_live < 1 or page_size < 1:
            raise ValueError("max_live and page_size must be >= 1")
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.max_live = max_live
        _, _, self.model = load_model(model_dir, dtype=self.dtype, device=self.device)
        spec = self.model.spec
        pages = max(1, pages_for(max_tokens, page_size))
        max_seq_len = min(spec.max_positions, pages * page_size)
        self.cache = CacheManager(self.model.cache_needs(), num_pages=pages, num_slots=max_live,
                                  max_seq_len=max_seq_len, page_size=page_size, dtype=self.dtype, device=self.device,
                                  enable_prefix_cache=False)
        self.runner = ModelRunner(self.model, self.cache, device=self.device, use_graphs=use_graphs)
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
                    raise EngineError(f"request {rid!r}: more than {self.max_live} requests are live (--max-live)")
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
            _check_status(self.dtype)
        for rid in record.get("end", []):
            slot = self.slot_of.pop(str(rid), None)
            if slot is not None:
                self.cache.close(slot)
        return out


def _check_status(dtype: torch.dtype) -> None:
    if dtype == torch.bfloat16:  # the device has just been waited for: see whether a bounded wait gave up
        status = library.tcgen05_status()
        if status:
            raise EngineError(f"a tcgen05 kernel gave up waiting on a barrier (status {status:#x}); results are void")


class ScheduledReplayer:
    """Scheduler mode: the trace says when requests arrive and what they generate; the scheduler decides the batches
    and the engine runs them as in ``LLM.generate`` (steps launched ahead, captured decode steps)."""

    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, device: str = "cuda", *,
                 max_seq_len: int | None = None, chunk: int = 512, max_running: int = 8, page_size: int = PAGE_SIZE,
                 prefix_cache: bool = True, ahead: bool = True, use_graphs: bool = True) -> None:
        from .engine import Engine, EngineConfig
        from .scheduler import Scheduler
        from ..config.registry import read_model_folder
        pages = max(1, pages_for(max_tokens, page_size))
        arch, config = read_model_folder(model_dir)
        max_seq_len = max_seq_len or min(pages * page_size, arch.to_spec(config).max_positions)
        self.engine = Engine(EngineConfig(
            model_path=Path(model_dir), dtype=parse_dtype(dtype), device=device, max_num_seqs=max_running,
            max_prefill_tokens=chunk, max_seq_len=max_seq_len, num_blocks=pages, page_size=page_size,
            enable_prefix_cache=prefix_cache, use_cuda_graphs=use_graphs))
        self.engine.capture_logits = True
        self.scheduler = Scheduler(self.engine.cache, chunk_size=chunk, stop_token_ids=(), enable_prefix_cache=prefix_cache)
        self.chunk, self.max_running, self.ahead = chunk, max_running, ahead
        self.forced: dict[str, list[int]] = {}
        self.prompt_len: dict[str, int] = {}
        self._pending = None  # a step launched ahead of the previous line's commit

    def _override(self, batch) -> dict[str, int]:
        """The tokens the trace gives for the positions this batch samples."""
        out = {}
        for w in batch.work:
            if w.samples:
                at = len(w.req.output) + (1 if w.ahead else 0)
                out[w.req.req_id] = self.forced[w.req.req_id][at]
        return out

    def run_step(self, record: dict) -> tuple[np.ndarray | None, dict]:
        """One scheduler step.  Returns (float32 [rows, vocab] or None, what the rows are and what else happened)."""
        from .scheduler import AddResult
        sched, engine = self.scheduler, self.engine
        for add in record.get("add", []):
            rid, forced = str(add["id"]), [int(t) for t in add["forced"]]
            if not forced:
                raise EngineError(f"request {rid!r}: a request must generate at least one token")
            verdict = sched.add_request(rid, add["prompt"], len(forced), ignore_eos=True)
            if verdict is not AddResult.ACCEPTED:
                raise EngineError(f"request {rid!r} was refused: {verdict.value}")
            self.forced[rid] = forced
            self.prompt_len[rid] = len(add["prompt"])
        for rid in record.get("abort", []):
            sched.free_request(str(rid))
        info: dict = {"rows": [], "preempted": [], "finished": {}}
        pending = self._pending
        if pending is None:
            if not sched.has_work():
                return None, info
            batch = sched.schedule_step(self.chunk, self.max_running)
            pending = engine.launch(batch, override=self._override(batch))
        self._pending = None
        if self.ahead:
            nxt = sched.schedule_ahead(self.max_running)
            if nxt is not None:
                self._pending = engine.launch(nxt, feed=pending, override=self._override(nxt))
        tokens = engine.finish(pending)
        rows = pending.logits.cpu().numpy().astype("<f4", copy=False) if pending.logits is not None else None
        for w in pending.sampling:
            info["rows"].append({"id": w.req.req_id, "position": w.end})
        result = sched.commit(pending.batch, tokens)
        info["preempted"] = list(pending.batch.preempted)
        info["finished"] = {rid: reason.value for rid, reason in result.finished.items()}
        _check_status(engine.dtype)
        return rows, info

    def counters(self) -> dict:
        st = self.scheduler.stats()
        return {"prompt_tokens": st.prompt_tokens, "cached_prompt_tokens": st.cached_prompt_tokens,
                "preemptions": st.preemptions, "launched_ahead": self.engine.launched_ahead,
                "graph_replays": self.engine.runner.graph_replays, "steps": self.engine.runner.steps_run,
                "free_blocks": st.free_blocks, "cached_blocks": st.cached_blocks}


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine, write logits")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time (sizes the pool)")
    p.add_argument("--mode", choices=["step", "scheduler"], default="step",
                   help="step: the trace names every batch; scheduler: the trace names arrivals, the scheduler batches")
    p.add_argument("--max-live", type=int, default=LIVE_REQUESTS, help="request slots (step mode)")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    p.add_argument("--no-graphs", action="store_true", help="run decode steps without captured CUDA graphs")
    p.add_argument("--max-seq-len", type=int, default=None, help="scheduler mode: longest request (default: the pool)")
    p.add_argument("--chunk", type=int, default=512, help="scheduler mode: token budget of a step and longest portion")
    p.add_argument("--max-running", type=int, default=8, help="scheduler mode: requests running at once")
    p.add_argument("--no-prefix-cache", action="store_true", help="scheduler mode: no prefix reuse")
    p.add_argument("--no-ahead", action="store_true", help="scheduler mode: wait for every step before the next")
    args = p.parse_args(argv)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    if args.mode == "step":
        replayer = Replayer(args.model, args.dtype, args.max_tokens, max_live=args.max_live, page_size=args.page_size,
                            use_graphs=not args.no_graphs)
    else:
        replayer = ScheduledReplayer(args.model, args.dtype, args.max_tokens, max_seq_len=args.max_seq_len, chunk=args.chunk,
                                     max_running=args.max_running, page_size=args.page_size,
                                     prefix_cache=not args.no_prefix_cache, ahead=not args.no_ahead,
                                     use_graphs=not args.no_graphs)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        if args.mode == "step":
            logits = replayer.run_step(record)
        else:
            logits, info = replayer.run_step(record)
            (out_dir / f"{step}.json").write_text(json.dumps(info))
        if logits is not None and logits.shape[0] > 0:
            logits.tofile(out_dir / f"{step}.f32")
        print(f"done {step}", flush=True)
    if args.mode == "scheduler":
        print("stats " + json.dumps(replayer.counters()), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
