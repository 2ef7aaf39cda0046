"""The engine: a model folder, a cache and the step function, driven by batches
of the scheduler.

Mirrors what the reference's engine offers a driver
(prefixserve/engine.py:10-29, prefixserve/llama_engine.py:46-150):
``num_blocks``, ``max_seq_len``, ``stop_token_ids`` and a blocking
``step(batch) -> {request id: token}``; the pool is sized from free memory
after a worst-case trial step when ``num_blocks`` is not given
(prefixserve/llama_engine.py:231-267).
"""

from __future__ import annotations

import gc
import logging
from dataclasses import dataclass, replace
from pathlib import Path

import numpy as np
import torch

from ..cache.manager import CacheManager, pages_for
from ..config.registry import read_model_folder
from .loading import load_model, parse_dtype
from .scheduler import Batch
from .step import EngineError, ModelRunner, StepItem

log = logging.getLogger(__name__)


@dataclass(frozen=True)
class EngineConfig:
    model_path: Path
    dtype: torch.dtype = torch.bfloat16
    device: str = "cuda"
    max_num_seqs: int = 64           # must match the scheduler's max_decode_seqs
    max_prefill_tokens: int = 512    # must match the scheduler's budget
    max_seq_len: int | None = None   # None: the smaller of 8192 (the reference's default) and the model's positions
    num_blocks: int | None = None    # pages of every cache group; None: size the pools from free memory
    reserve_bytes: int = 1 << 30     # left free after the pool
    page_size: int = 16
    enable_prefix_cache: bool = True
    use_cuda_graphs: bool = True     # capture pure-decode steps per batch size and replay them
    cast_float32_weights: bool = False  # round matrices a checkpoint stores in 32-bit to the compute type at load


@dataclass
class PendingStep:
    """A step that has been put on the device: what ``Engine.finish`` needs to hand out its tokens, and what a step
    launched right behind it needs to take its input tokens from."""
    batch: Batch
    sampling: list                       # the work items that sample, in the order of the tokens
    tokens_dev: torch.Tensor | None      # int32 [len(sampling)] on the device
    host: torch.Tensor | None            # the same in pinned host memory once ``done`` has passed
    done: torch.cuda.Event | None
    logits: torch.Tensor | None = None   # with ``Engine.capture_logits``: float32 [len(sampling), vocab], a copy on the device


class Engine:
    def __init__(self, cfg: EngineConfig) -> None:
        self.cfg = cfg
        self.device = torch.device(cfg.device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise EngineError("no CUDA device: this engine has no CPU path")
        dtype = parse_dtype(cfg.dtype)
        arch, model_cfg = read_model_folder(cfg.model_path)
        positions = arch.to_spec(model_cfg).max_positions
        if cfg.max_seq_len is None:
            cfg = self.cfg = replace(cfg, max_seq_len=min(8192, positions))
        elif cfg.max_seq_len > positions:
            raise ValueError(f"max_seq_len {cfg.max_seq_len} exceeds the model's {positions} positions")
        self.arch, self.model_cfg, self.model = load_model(cfg.model_path, dtype=dtype, device=self.device,
                                                           max_positions=cfg.max_seq_len,
                                                           cast_float32=cfg.cast_float32_weights)
        self.dtype = dtype
        self.needs = self.model.cache_needs()
        self.bytes_per_block = CacheManager.bytes_per_page(self.needs, cfg.page_size, dtype)
        num_blocks = cfg.num_blocks if cfg.num_blocks is not None else self._size_pool()
        self.cache = self._make_cache(num_blocks)
        self.runner = ModelRunner(self.model, self.cache, device=self.device, use_graphs=cfg.use_cuda_graphs, sample=True)
        self.capture_logits = False
        self.last_logits: dict[str, torch.Tensor] = {}
        # sampled tokens come back through pinned host memory; two buffers, because a step may be launched while the
        # one before it has not been read yet
        self._token_buffers = [torch.empty(cfg.max_num_seqs, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._token_turn = 0
        self.launched_ahead = 0  # steps launched before the step in front of them had been read
        log.info("cache: %s pages of %d tokens", num_blocks, cfg.page_size)

    def _make_cache(self, num_blocks) -> CacheManager:
        return CacheManager(self.needs, num_pages=num_blocks, num_slots=self.cfg.max_num_seqs,
                            max_seq_len=self.cfg.max_seq_len, page_size=self.cfg.page_size, dtype=self.dtype,
                            device=self.device, enable_prefix_cache=self.cfg.enable_prefix_cache)

    # ---- what a driver needs ------------------------------------------------
    @property
    def num_blocks(self) -> int:
        return self.cache.num_pages(0)

    @property
    def max_seq_len(self) -> int:
        return self.cfg.max_seq_len

    def weight_bytes(self) -> int:
        """Bytes of the loaded weights, a tied head counted once."""
        return self.model.num_bytes()

    @property
    def stop_token_ids(self) -> frozenset[int]:
        return self.model.spec.stop_token_ids

    @torch.inference_mode()
    def step(self, batch: Batch) -> dict[str, int]:
        """Runs one batch of the scheduler; returns request id -> next token for the items that sample."""
        return self.finish(self.launch(batch))

    @torch.inference_mode()
    def launch(self, batch: Batch, feed: "PendingStep | None" = None,
               override: "dict[str, int] | None" = None) -> "PendingStep":
        """Puts one batch on the device (forward, sampling, copy of the tokens to pinned host memory) and returns
        without waiting for it.  ``feed``: the step launched just before, not finished yet, whose sampled tokens are
        this batch's input tokens (a batch from ``Scheduler.schedule_ahead``); they go from its output to this step's
        input on the device.  ``override`` (request id -> token): these tokens stand in for the sampled ones, on the
        device too, so that a step fed from this one continues with them (teacher forcing, as the reference's tests
        do at commit: tests/gpu/test_engine_flashinfer.py:50-77 of PrefixServe)."""
        work = batch.work
        if not work:
            return PendingStep(batch, [], None, None, None)
        if len(work) > self.cfg.max_num_seqs or batch.num_tokens > self.cfg.max_prefill_tokens + self.cfg.max_num_seqs:
            raise EngineError(f"batch of {len(work)} requests / {batch.num_tokens} tokens is over the engine's limits")
        ahead = any(w.ahead for w in work)
        device_ids = None
        if ahead:
            if feed is None or feed.tokens_dev is None or not all(w.ahead for w in work) or \
                    [w.req for w in work] != [w.req for w in feed.sampling]:
                raise EngineError("a batch scheduled ahead must follow, request by request, the step that feeds it")
            device_ids = feed.tokens_dev
            self.launched_ahead += 1
            placeholder = np.zeros(1, dtype=np.int32)
            items = [StepItem(w.req.slot, w.start, placeholder, (0,)) for w in work]
        else:
            items = [StepItem(w.req.slot, w.start, w.req.tokens(w.start, w.end), (w.end - w.start - 1,) if w.samples else ())
                     for w in work]
        in_flight = [w.end - w.start for w in feed.sampling] if ahead else None
        logits = self.runner.step(items, device_ids=device_ids, in_flight=in_flight)
        sampling = [w for w in work if w.samples]
        if not sampling:
            return PendingStep(batch, [], None, None, None)  # nothing to read back: the host runs ahead
        tokens = self.runner.last_tokens  # chosen inside the step (and inside its capture, where it has one)
        if override is not None:
            given = [override.get(w.req.req_id) for w in sampling]
            if all(g is not None for g in given):
                tokens = torch.tensor(given, dtype=torch.int32).to(self.device, non_blocking=True)
            elif any(g is not None for g in given):
                mask = torch.tensor([g is not None for g in given]).to(self.device)
                tokens = torch.where(mask, torch.tensor([g or 0 for g in given], dtype=torch.int32).to(self.device), tokens)
        kept = logits.clone() if self.capture_logits else None  # a replayed graph's logits last until its next replay
        host = self._token_buffers[self._token_turn % len(self._token_buffers)][: len(sampling)]
        self._token_turn += 1
        host.copy_(tokens, non_blocking=True)  # the step's one device-to-host read
        done = torch.cuda.Event()
        done.record()
        return PendingStep(batch, sampling, tokens, host, done, kept)

    def finish(self, pending: "PendingStep") -> dict[str, int]:
        """Waits for a launched step; returns request id -> next token for the items that sample."""
        if pending.done is None:
            return {}
        pending.done.synchronize()
        if pending.logits is not None:
            rows = pending.logits.cpu()
            self.last_logits = {w.req.req_id: rows[i] for i, w in enumerate(pending.sampling)}
        return {w.req.req_id: tok for w, tok in zip(pending.sampling, pending.host.tolist())}

    def check_device_status(self) -> None:
        """Raises if a bounded wait inside a tensor-core kernel ever gave up on this device: the results of that launch
        (and possibly of later ones) are void.  Reading the status waits for the device, so callers do it where they
        wait anyway: at the end of a generate call, at the end of a replay."""
        from ..ops import library
        status = library.tcgen05_status()
        if status:
            raise EngineError(f"a tcgen05 kernel gave up waiting on a barrier (status {status:#x}); results are void")

    def capture_decode_graphs(self, batch_sizes) -> int:
        """Captures the pure-decode step for the given batch sizes and every class of sequence lengths now, so that no
        request pays for a capture (a few milliseconds each) in the middle of serving.  Needs the cache to have that
        many free slots and pages.  Returns how many graphs were captured."""
        if not self.runner.use_graphs:
            return 0
        done = 0
        for b in sorted(set(int(x) for x in batch_sizes)):
            if b < 1 or b > self.cfg.max_num_seqs:
                continue
            if self.cache.slots.num_free < b or self.cache.free_pages(0) < b:
                break
            wanted = [k for k in self.runner.length_classes if not self.runner.has_decode_graph(b, k)]
            if not wanted:
                continue
            slots = []
            for _ in range(b):
                slot = self.cache.open()
                self.cache.reserve(slot, 1)
                slots.append(slot)
            for klass in wanted:  # each call runs the step, then captures it
                self.runner.step([StepItem(s, 0, np.zeros(1, dtype=np.int32), (0,)) for s in slots], length_class=klass)
                done += 1
            for s in slots:
                self.cache.close(s)
        torch.cuda.synchronize()
        return done

    def graph_bytes_estimate(self) -> int:
        """What the captured decode steps of every batch size and length class keep for themselves: their logits."""
        if not self.cfg.use_cuda_graphs:
            return 0
        n = self.cfg.max_num_seqs
        classes = len(ModelRunner._length_classes(self.cfg.max_seq_len))
        return classes * (n * (n + 1) // 2) * self.model.spec.vocab_size * 4

    # ---- pool sizing ----------------------------------------------------------
    def _size_pool(self) -> int:
        """Pages that fit beside the weights and the activations of a worst-case step."""
        cfg = self.cfg
        prefill = min(cfg.max_prefill_tokens, cfg.max_seq_len)
        trial_pages = pages_for(prefill, cfg.page_size) + cfg.max_num_seqs
        torch.cuda.synchronize()
        gc.collect()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        before = torch.cuda.memory_allocated()
        cache = self._make_cache(trial_pages)
        runner = ModelRunner(self.model, cache, device=self.device, use_graphs=False)
        held = torch.cuda.memory_allocated() - before
        items = []
        for i in range(cfg.max_num_seqs):
            n = prefill if i == 0 else 1
            slot = cache.open()
            cache.reserve(slot, n)
            items.append(StepItem(slot, 0, np.zeros(n, dtype=np.int32), (n - 1,)))
        runner.step(items)
        torch.cuda.synchronize()
        activations = torch.cuda.max_memory_allocated() - before - held
        cache.release_device_memory()  # the trial pages go back before the real pool is measured for
        del cache, runner
        gc.collect()
        torch.cuda.empty_cache()
        free, _ = torch.cuda.mem_get_info()
        usable = free - activations - cfg.reserve_bytes - self.graph_bytes_estimate()
        # Groups with a window are given what every running request can hold at once (the window, a portion and a
        # page of slack); what is left goes to the groups that keep all keys, which share it page for page.
        by_group = CacheManager.group_page_bytes(self.needs, cfg.page_size, self.dtype)
        sizes: dict[int, int] = {}
        for gi, (window, cost) in enumerate(by_group.items()):
            if window is not None:
                sizes[gi] = cfg.max_num_seqs * (pages_for(min(cfg.max_seq_len, window + prefill), cfg.page_size) + 1)
                usable -= sizes[gi] * cost
        full_cost = sum(cost for window, cost in by_group.items() if window is None)
        need = pages_for(cfg.max_seq_len, cfg.page_size)
        if full_cost:
            n = int(usable // full_cost)
            if n < need:
                raise EngineError(f"only {n} cache pages fit ({usable / 1e9:.2f} GB usable); one request of max_seq_len needs {need}")
            for gi, window in enumerate(by_group):
                if window is None:
                    sizes[gi] = n
        elif usable < 0:
            raise EngineError(f"the windowed cache groups alone do not fit ({-usable / 1e9:.2f} GB short)")
        log.info("trial step: activations %.0f MB, %.2f GB free -> pages per group %s", activations / 1e6, free / 1e9, sizes)
        return sizes if len(sizes) != 1 else next(iter(sizes.values()))
