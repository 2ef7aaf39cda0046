"""The step function: one batch of (request, its next tokens) through the model.

A batch mixes portions of prompts with single decoded tokens, cut anywhere.
Only the given tokens are computed; everything earlier is read from the cache.
The result is the float32 logits at the positions the caller asks for.

Host work per step, after the reference (prefixserve/llama_engine.py:152-227):
all integer inputs are laid out in one pinned buffer and reach the device in a
single asynchronous copy; page tables and limits are checked on the host
before anything is launched (prefixserve/llama_engine.py:270-287), so a bad
table is an exception for one step, not a memory fault.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, pages_for
from ..parts.base import ItemView, StepContext
from ..ops import library
from ..parts.model import DecoderModel


class EngineError(RuntimeError):
    """The step function was given a batch it cannot run."""


@dataclass
class StepItem:
    slot: int
    start: int                       # absolute position of the first token
    tokens: np.ndarray               # int32, the next tokens of the request
    want: Sequence[int] = field(default_factory=tuple)  # offsets into tokens whose logits are wanted


@dataclass
class _DecodeGraph:
    """A captured pure-decode step for one batch size: fixed input buffer, fixed output, the graph."""

    inputs: torch.Tensor
    logits: torch.Tensor
    graph: torch.cuda.CUDAGraph
    kernels: int = 0  # launches of this library's kernels recorded in the graph


class ModelRunner:
    """Owns the per-step staging buffers and runs ``DecoderModel.forward`` on the cache.

    Steps in which every item brings one token and wants its logits are
    launch-bound (some hundred small kernels); they are captured once per
    batch size as a CUDA graph over a fixed input buffer and replayed.  The
    logits of such a step live in the graph's own memory and are valid until
    the next step of the same batch size.
    """

    def __init__(self, model: DecoderModel, cache: CacheManager, *, device: torch.device | str,
                 use_graphs: bool = True) -> None:
        if model.compute_dtype is None:
            raise EngineError("the model has no weights yet")
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise EngineError(f"the engine runs on a CUDA device only, not on {self.device}")
        self.vocab_size = model.spec.vocab_size
        self._host: torch.Tensor | None = None
        self._copied = torch.cuda.Event()
        self._copy_pending = False
        self.steps_run = 0
        self.last_h2d_bytes = 0  # size of the last step's single host-to-device copy
        # graphs need every part to do the same device work for the same shapes, whatever the host-side item list says
        self.use_graphs = use_graphs and all(getattr(p, "graph_safe", False) for _, p in model.named_parts())
        self._graphs: dict[int, _DecodeGraph] = {}
        self._graph_pool = None  # one memory pool for all captured steps: only one of them runs at a time
        self.graph_replays = 0
        # Test-only, after the reference's EngineConfig.inject_bug (prefixserve/llama_engine.py:62-63, :192, :202-203):
        # "rope_relative" numbers every portion's positions from 0; "kv_len_short" reports one key too few.
        # The test suite proves with these that it notices such faults.
        self.inject_bug: str | None = None

    # ------------------------------------------------------------------ checks
    def _check(self, items: Sequence[StepItem], ahead: np.ndarray | None = None) -> None:
        seen: set[int] = set()
        for at, it in enumerate(items):
            n = len(it.tokens)
            if n < 1:
                raise EngineError(f"slot {it.slot}: an item needs at least one token")
            if it.slot in seen:
                raise EngineError(f"slot {it.slot} appears twice in one step")
            seen.add(it.slot)
            if not self.cache.slots.taken(it.slot):
                raise EngineError(f"slot {it.slot} is not open")
            if it.start != self.cache.position(it.slot) + (0 if ahead is None else int(ahead[at])):
                raise EngineError(f"slot {it.slot}: tokens start at {it.start} but the cache holds {self.cache.position(it.slot)}")
            end = it.start + n
            if end > self.cache.max_seq_len:
                raise EngineError(f"slot {it.slot}: position {end} exceeds max_seq_len {self.cache.max_seq_len}")
            if self.cache.shortfall(it.slot, end):
                raise EngineError(f"slot {it.slot}: no pages reserved for positions up to {end}")
            for w in it.want:
                if not 0 <= w < n:
                    raise EngineError(f"slot {it.slot}: wanted offset {w} outside its {n} tokens")
        every = np.concatenate([np.asarray(it.tokens).reshape(-1) for it in items])  # one pass instead of one per item
        if every.min() < 0 or every.max() >= self.vocab_size:
            bad = next(it.slot for it in items if np.min(it.tokens) < 0 or np.max(it.tokens) >= self.vocab_size)
            raise EngineError(f"slot {bad}: token id outside [0, {self.vocab_size})")

    def _check_tables(self, items: Sequence[StepItem], tables: dict[int, np.ndarray]) -> None:
        page = self.cache.page_size
        for gi, table in tables.items():
            g = self.cache.groups[gi]
            for row, it in zip(table, items):
                end = it.start + len(it.tokens)
                first = self.cache._first_needed_page(g, it.start)
                live = row[first: pages_for(end, page)]
                if live.size and (live.min() < 0 or live.max() >= g.pool.num_blocks):
                    raise EngineError(f"slot {it.slot}: page table of group {gi} names a page outside the pool")

    # ------------------------------------------------------------------- step
    @torch.inference_mode()
    def step(self, items: Sequence[StepItem], device_ids: torch.Tensor | None = None,
             in_flight: Sequence[int] | None = None) -> torch.Tensor:
        """Runs the batch. Returns float32 logits [number of wanted positions, vocab] on the device,
        in the order of the items and of each item's ``want``.

        ``device_ids`` (int32 [len(items)] on the device): the items are single tokens that follow a step which has been
        launched but whose result the host has not seen; their token ids are taken from this tensor on the device (the
        items' own ``tokens`` are placeholders); ``in_flight[i]`` is how many tokens that step computes for item i's
        request, which the cache manager does not record before its commit."""
        if not items:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        ahead = None
        if device_ids is not None:
            if any(len(it.tokens) != 1 for it in items) or device_ids.numel() != len(items) or device_ids.dtype != torch.int32 \
                    or not device_ids.is_cuda or in_flight is None or len(in_flight) != len(items):
                raise EngineError("token ids from the device: one int32 per item, every item a single token")
            ahead = np.asarray(in_flight, dtype=np.int64)
        held = self._graphs.get(len(items)) if self.use_graphs else None
        if held is not None and all(len(it.tokens) == 1 and tuple(it.want) == (0,) for it in items):
            return self._replay(items, held, device_ids, ahead)
        self._check(items, ahead)
        lens = [len(it.tokens) for it in items]
        b, t = len(items), sum(lens)
        s = sum(len(it.want) for it in items)
        page = self.cache.page_size
        static = self.use_graphs and t == b and all(tuple(it.want) == (0,) for it in items)
        if static:  # the shapes of a captured step may not depend on the step: full-width page tables
            widths = {gi: self.cache.max_pages_per_seq for gi in range(len(self.cache.groups))}
        else:
            widths = {gi: max(pages_for(it.start + n, page) for it, n in zip(items, lens))
                      for gi in range(len(self.cache.groups))}
        tables = self.cache.tables_for([it.slot for it in items], widths)
        self._check_tables(items, tables)

        # layout of the one staging buffer (int32 words)
        o_ids, o_pos, o_item = 0, t, 2 * t
        o_start = 3 * t
        o_kvlen = o_start + b + 1
        o_slot = o_kvlen + b
        o_rows = o_slot + b
        o_tab = o_rows + s
        total = o_tab + sum(b * w for w in widths.values())

        host = self._staging(total)
        buf = host.numpy()
        views: list[ItemView] = []
        tok = ri = 0
        buf[o_start] = 0
        for i, (it, n) in enumerate(zip(items, lens)):
            buf[o_ids + tok: o_ids + tok + n] = it.tokens
            first = 0 if self.inject_bug == "rope_relative" else it.start
            buf[o_pos + tok: o_pos + tok + n] = np.arange(first, first + n, dtype=np.int32)  # absolute positions
            buf[o_item + tok: o_item + tok + n] = i
            buf[o_kvlen + i] = it.start + n - (1 if self.inject_bug == "kv_len_short" and it.start + n > n else 0)
            buf[o_slot + i] = it.slot
            for w in it.want:
                buf[o_rows + ri] = tok + w
                ri += 1
            views.append(ItemView(slot=it.slot, start=it.start, end=it.start + n, first_token=tok))
            tok += n
            buf[o_start + i + 1] = tok
        at = o_tab
        table_at: dict[int, tuple[int, int]] = {}
        for gi, table in tables.items():
            w = widths[gi]
            buf[at: at + b * w] = table.reshape(-1)
            table_at[gi] = (at, w)
            at += b * w

        self.last_h2d_bytes = 4 * total
        if static:
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
            dev.copy_(host[:total], non_blocking=True)
        else:
            dev = host[:total].to(self.device, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        if device_ids is not None:
            dev[o_ids: o_ids + t].copy_(device_ids)

        ctx = StepContext(
            num_tokens=t,
            num_items=b,
            compute_dtype=self.model.compute_dtype,
            device=self.device,
            items=views,
            token_ids=dev[o_ids: o_ids + t],
            positions=dev[o_pos: o_pos + t],
            token_item=dev[o_item: o_item + t],
            item_start=dev[o_start: o_start + b + 1],
            kv_len=dev[o_kvlen: o_kvlen + b],
            slots=dev[o_slot: o_slot + b],
            block_tables={gi: dev[a: a + b * w].view(b, w) for gi, (a, w) in table_at.items()},
            max_new_tokens=max(lens),
            max_kv_len=max(it.start + n for it, n in zip(items, lens)),
            all_decode=all(n == 1 for n in lens),
        )
        if static:
            ctx.extras["static_kv_len"] = self.cache.max_seq_len
        rows = dev[o_rows: o_rows + s]
        with library.pinned_stream():  # one look-up of the stream for the step's hundred-odd launches
            logits = self.model.forward(ctx, self.cache.view, rows)  # this step's result, computed eagerly
        self.steps_run += 1
        if static:
            # Capture the same launches for later steps of this batch size.  Nothing runs during capture; the eager
            # run above has already sized every scratch buffer the kernels use.
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = library.launches
            with torch.cuda.graph(graph, pool=self._graph_pool):
                with library.pinned_stream():  # the capture's own stream
                    static_logits = self.model.forward(ctx, self.cache.view, rows)
            self._graphs[b] = _DecodeGraph(inputs=dev, logits=static_logits, graph=graph, kernels=library.launches - before)
            library.launches = before  # recorded, not run
        return logits

    def _replay(self, items: Sequence[StepItem], held: _DecodeGraph, device_ids: torch.Tensor | None = None,
                ahead: np.ndarray | None = None) -> torch.Tensor:
        """A pure-decode step of a batch size that has been captured: the same checks and the same buffer layout as
        the general path, written with array operations instead of per-item loops, then one copy and one replay."""
        cache = self.cache
        b = len(items)
        slots = np.fromiter((it.slot for it in items), dtype=np.int32, count=b)
        starts = np.fromiter((it.start for it in items), dtype=np.int64, count=b)
        toks = np.fromiter((it.tokens[0] for it in items), dtype=np.int64, count=b)
        if len(set(slots.tolist())) != b:
            raise EngineError("a slot appears twice in one step")
        if slots.min() < 0 or slots.max() >= cache.num_slots or not all(cache.slots.taken(int(s)) for s in slots):
            raise EngineError("a slot of the step is not open")
        if not np.array_equal(starts, cache._position[slots] + (0 if ahead is None else ahead)):
            raise EngineError("tokens do not start where the cache ends for some slot of the step")
        if starts.max() + 1 > cache.max_seq_len:
            raise EngineError(f"a position exceeds max_seq_len {cache.max_seq_len}")
        if toks.min() < 0 or toks.max() >= self.vocab_size:
            raise EngineError(f"token id outside [0, {self.vocab_size})")
        page = cache.page_size
        need = (starts + page) // page  # pages that must be held to cover position `start`
        width = cache.max_pages_per_seq
        t = s = b
        o_ids, o_pos, o_item, o_start = 0, t, 2 * t, 3 * t
        o_kvlen = o_start + b + 1
        o_slot = o_kvlen + b
        o_rows = o_slot + b
        o_tab = o_rows + s
        total = o_tab + len(cache.groups) * b * width
        host = self._staging(total)
        buf = host.numpy()
        cols = np.arange(width)[None, :]
        at = o_tab
        for gi, g in enumerate(cache.groups):
            table = buf[at: at + b * width].reshape(b, width)
            g.tables.gather(slots, width, table)
            first = 0 if g.window is None else np.maximum(0, starts - g.window + 1)[:, None] // page
            live = (cols >= first) & (cols < need[:, None])
            if (live & ((table < 0) | (table >= g.pool.num_blocks))).any():
                raise EngineError(f"a page table of group {gi} lacks a page or names one outside the pool")
            at += b * width
        ramp = np.arange(b + 1, dtype=np.int32)
        buf[o_ids: o_ids + b] = toks
        buf[o_pos: o_pos + b] = 0 if self.inject_bug == "rope_relative" else starts
        buf[o_item: o_item + b] = ramp[:b]
        buf[o_start: o_start + b + 1] = ramp
        buf[o_kvlen: o_kvlen + b] = starts + 1 - (1 if self.inject_bug == "kv_len_short" else 0) * (starts > 0)
        buf[o_slot: o_slot + b] = slots
        buf[o_rows: o_rows + b] = ramp[:b]
        self.last_h2d_bytes = 4 * total
        held.inputs.copy_(host[:total], non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        if device_ids is not None:
            held.inputs[o_ids: o_ids + b].copy_(device_ids)
        held.graph.replay()
        library.launches += held.kernels  # this library's kernels inside the replayed graph
        self.steps_run += 1
        self.graph_replays += 1
        return held.logits

    def _staging(self, words: int) -> torch.Tensor:
        # the previous step's copy must have left the buffer before it is overwritten
        if self._copy_pending:
            self._copied.synchronize()
            self._copy_pending = False
        if self._host is None or self._host.numel() < words:
            size = max(4096, 1 << (words - 1).bit_length())
            self._host = torch.empty(size, dtype=torch.int32, pin_memory=True)
        return self._host
