"""The step function: one batch of (request, its next tokens) through the model.

A batch mixes portions of prompts with single decoded tokens, cut anywhere.
Only the given tokens are computed; everything earlier is read from the cache.
The result is the float32 logits at the positions the caller asks for.

Host work per step, after the reference (prefixserve/llama_engine.py:152-227):
all integer inputs are laid out in one pinned buffer and reach the device in a
single asynchronous copy; page tables and limits are checked on the host
before anything is launched (prefixserve/llama_engine.py:270-287), so a bad
table is an exception for one step, not a memory fault.

Unlike the reference, which flattens and uploads every request's page list on
every step (prefixserve/llama_engine.py:183-209), the page tables and a record
per request slot (position, sampling temperature and seed) stay on the device.
A step carries the words of them that changed since the last one as (index,
value) pairs behind its other inputs; a small kernel puts them in place and
another turns the rows of the step's slots into the table the layers read.  A
decode step that appends no page sends four words per request.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import os

import numpy as np
import torch

from ..cache.manager import CacheManager, pages_for
from ..parts.base import ItemView, StepContext
from .. import ops
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
    """A captured step for one shape (a batch size of single tokens, or a tuple of item lengths): fixed input buffer,
    fixed output, the graph."""

    inputs: torch.Tensor
    logits: torch.Tensor
    graph: torch.cuda.CUDAGraph
    var_at: int      # where the words that change from step to step begin in ``inputs``
    pairs_at: int    # where the (index, value) pairs of the resident array begin
    pairs_room: int  # how many pairs fit
    kernels: int = 0  # launches of this library's kernels recorded in the graph
    by_name: dict | None = None  # the same by entry point
    layout: "_Layout | None" = None
    tokens: torch.Tensor | None = None  # with sampling inside the step: int32 [wanted rows], the chosen tokens


@dataclass
class _Layout:
    """Where each input of a step lies in its one int32 buffer.  What never changes between steps of the same shape
    comes first, what changes next, the changed words of the resident array last."""

    t: int
    b: int
    s: int
    rows_are_items: bool = False  # every item brings one token and wants it: the slot of a row is the slot of its item

    def __post_init__(self) -> None:
        t, b, s = self.t, self.b, self.s
        self.item, self.start, self.rows = 0, t, t + b + 1
        self.var = self.rows + s
        self.ids, self.pos, self.kvlen = self.var, self.var + t, self.var + 2 * t
        self.slot = self.kvlen + b
        self.rowslot = self.slot if self.rows_are_items else self.slot + b
        self.pairs = self.rowslot + s


class ModelRunner:
    """Owns the per-step staging buffers and runs ``DecoderModel.forward`` on the cache.

    Steps in which every item brings one token and wants its logits are
    launch-bound (some hundred small kernels); they are captured once per
    batch size as a CUDA graph over a fixed input buffer and replayed.  The
    logits of such a step live in the graph's own memory and are valid until
    the next step of the same batch size.

    Steps with prompt portions of up to a thousand tokens are bound by the
    host too (a step's launches take the host about two milliseconds, the
    device less).  Their shape is the tuple of the items' lengths with, per
    item, whether the last position's logits are wanted; a shape that comes a
    second time is captured and replayed from then on (a long prompt cut into
    equal portions, a portion beside the same decoding requests step after
    step).  Everything that varies inside a shape (tokens, positions, lengths
    of the cached prefixes, slots) is device data.
    """

    def __init__(self, model: DecoderModel, cache: CacheManager, *, device: torch.device | str,
                 use_graphs: bool = True, sample: bool = False) -> None:
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
        self.last_row_slots: torch.Tensor | None = None  # int32 [wanted rows]: the request slot of each row of the last logits
        # With ``sample`` every step also chooses a token for each wanted row (sampling/sampler.py: the temperature,
        # seed and position of the row's slot record), as part of the captured launches where the step is captured:
        # launched after a replay instead, the sampling kernels start only when the whole graph has drained.
        self.sample_in_step = sample
        self.last_tokens: torch.Tensor | None = None  # int32 [wanted rows] on the device (with ``sample``)
        # graphs need every part to do the same device work for the same shapes, whatever the host-side item list says
        self.use_graphs = use_graphs and all(getattr(p, "graph_safe", False) for _, p in model.named_parts())
        self._graphs: dict[tuple[int, int], _DecodeGraph] = {}  # pure-decode steps, by (batch size, length class)
        # A captured step's launch shapes (key ranges of attention, width of the page tables) cannot follow the
        # step's lengths, so they are sized for a class of lengths: the step's longest sequence rounded up to a power
        # of two (from 1,024), at most the longest the cache allows.  A batch of short sequences thus does not run
        # with the few, long key ranges that the longest possible sequence would need.
        self.length_classes = self._length_classes(cache.max_seq_len)
        self._graph_pool = None  # one memory pool for all captured steps: only one of them runs at a time
        self.graph_replays = 0
        self._shape_graphs: dict[tuple, _DecodeGraph] = {}  # steps with portions, by shape; oldest out first
        self._shapes_seen: dict[tuple, int] = {}
        self.max_shape_graphs = 48
        self.capture_shapes_from = 2      # a shape is captured when it comes for this many-th time
        self.longest_captured_portion = 1024  # longer portions keep the device busy longer than the host needs
        # Test-only, after the reference's EngineConfig.inject_bug (prefixserve/llama_engine.py:62-63, :192, :202-203):
        # "rope_relative" numbers every portion's positions from 0; "kv_len_short" reports one key too few.
        # The test suite proves with these that it notices such faults.
        self.inject_bug: str | None = None
        # Debug check, after the reference's test harness (tests/test_llama_exact.py:146-151 of PrefixServe): a step
        # must never write a position whose page the prefix tree owns (another request may be reading it).
        self.check_writes = os.environ.get("PSB200_DEBUG_CHECKS", "0") == "1"

    @staticmethod
    def _length_classes(max_seq_len: int, smallest: int = 1024) -> tuple[int, ...]:
        out = []
        n = smallest
        while n < max_seq_len:
            out.append(n)
            n *= 2
        out.append(max_seq_len)
        return tuple(out)

    def length_class(self, longest: int) -> int:
        """The smallest length class that holds a sequence of ``longest`` tokens."""
        for n in self.length_classes:
            if longest <= n:
                return n
        raise EngineError(f"a position exceeds max_seq_len {self.cache.max_seq_len}")

    def has_decode_graph(self, batch_size: int, longest: int = 1) -> bool:
        return (batch_size, self.length_class(longest)) in self._graphs

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

    def _check_pages(self, slots: np.ndarray, starts: np.ndarray, ends: np.ndarray) -> None:
        """Every page a step reads or writes must be held and name a page of the pool; with the debug check on, no
        page it writes may belong to the prefix tree."""
        cache = self.cache
        page = cache.page_size
        upto = ((ends + page - 1) // page).astype(np.int32)
        for gi, g in enumerate(cache.groups):
            if g.window is None:
                first = np.zeros(len(slots), dtype=np.int32)
            else:
                first = (np.maximum(0, starts - g.window + 1) // page).astype(np.int32)
            bad = cache.covered(gi, slots, first, upto)
            if bad >= 0:
                raise EngineError(f"slot {int(slots[bad])}: page table of group {gi} lacks a page or names one outside the pool")
        if self.check_writes and cache.tree is not None:
            for slot, a, e in zip(slots.tolist(), starts.tolist(), ends.tolist()):
                row = cache.page_ids(slot)
                for pi in range(a // page, (e - 1) // page + 1):
                    if cache.is_cached(row[pi]):
                        raise EngineError(f"slot {slot}: the step would write position {max(a, pi * page)}, whose page "
                                          f"{row[pi]} belongs to the prefix cache")

    # -------------------------------------------------------- resident arrays
    def _send_deltas_alone(self) -> None:
        """Sends the changed words of the resident array in a copy of their own (when they do not fit behind a
        captured step's inputs)."""
        n = self.cache.pending_deltas()
        if n == 0:
            return
        host = self._staging(2 * n)
        n = self.cache.drain_deltas(host.numpy(), 0)
        dev = host[: 2 * n].to(self.device, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        ops.scatter_words(self.cache.resident, dev, n)

    def _device_step(self, lay: _Layout, dev: torch.Tensor, widths: dict[int, int], views, lens, static: int | None, rows: torch.Tensor):
        """The device work of a step whose inputs lie in ``dev``: the step's page tables from the resident rows, the
        slots' positions, then the model.  The same launches whether run at once or captured.  ``static``: the length
        class the launch shapes are sized for (a step that is captured), or None (shapes from the step's own lengths)."""
        cache = self.cache
        t, b = lay.t, lay.b
        kv_len = dev[lay.kvlen: lay.kvlen + b]
        slots = dev[lay.slot: lay.slot + b]
        tables: dict[int, torch.Tensor] = {}
        noted = False
        for gi in range(len(cache.groups)):
            tables[gi] = torch.empty((b, widths[gi]), dtype=torch.int32, device=self.device)
            ops.step_prepare(None if noted else cache.records_dev, kv_len, slots, cache.tables_dev[gi], tables[gi])
            noted = True
        if not noted:
            ops.step_prepare(cache.records_dev, kv_len, slots, None, None)
        ctx = StepContext(
            num_tokens=t,
            num_items=b,
            compute_dtype=self.model.compute_dtype,
            device=self.device,
            items=views,
            token_ids=dev[lay.ids: lay.ids + t],
            positions=dev[lay.pos: lay.pos + t],
            token_item=dev[lay.item: lay.item + t],
            item_start=dev[lay.start: lay.start + b + 1],
            kv_len=kv_len,
            slots=slots,
            block_tables=tables,
            max_new_tokens=max(lens),
            max_kv_len=max(v.end for v in views),
            all_decode=all(n == 1 for n in lens),
        )
        if static is not None:
            ctx.extras["static_kv_len"] = static
        return self.model.forward(ctx, cache.view, rows)

    # ------------------------------------------------------------------- step
    @torch.inference_mode()
    def step(self, items: Sequence[StepItem], device_ids: torch.Tensor | None = None,
             in_flight: Sequence[int] | None = None, length_class: int | None = None) -> torch.Tensor:
        """Runs the batch. Returns float32 logits [number of wanted positions, vocab] on the device,
        in the order of the items and of each item's ``want``; ``last_row_slots`` then names the slot of each row.
        The logits of a replayed step live in the capture's own buffer: they hold until the next step.

        ``length_class``: size a captured step for this class of sequence lengths instead of the smallest that holds
        the step (to capture a class before any sequence has grown into it).

        ``device_ids`` (int32 [len(items)] on the device): the items are single tokens that follow a step which has been
        launched but whose result the host has not seen; their token ids are taken from this tensor on the device (the
        items' own ``tokens`` are placeholders); ``in_flight[i]`` is how many tokens that step computes for item i's
        request, which the cache manager does not record before its commit."""
        if not items:
            self.last_row_slots = torch.empty(0, dtype=torch.int32, device=self.device)
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        ahead = None
        if device_ids is not None:
            if any(len(it.tokens) != 1 for it in items) or device_ids.numel() != len(items) or device_ids.dtype != torch.int32 \
                    or not device_ids.is_cuda or in_flight is None or len(in_flight) != len(items):
                raise EngineError("token ids from the device: one int32 per item, every item a single token")
            ahead = np.asarray(in_flight, dtype=np.int64)
        all_single = all(len(it.tokens) == 1 and tuple(it.want) == (0,) for it in items)
        # (a step that reaches beyond max_seq_len is refused by the checks below, whichever path it takes)
        klass = self.length_class(min(self.cache.max_seq_len, max(it.start + len(it.tokens) for it in items)))
        if length_class is not None:
            if length_class not in self.length_classes or length_class < klass:
                raise EngineError(f"length class {length_class} is none of {self.length_classes} or too short for the step")
            klass = length_class
        held = self._graphs.get((len(items), klass)) if self.use_graphs and all_single else None
        if held is not None:
            return self._replay(items, held, device_ids, ahead)
        shape = None
        if self.use_graphs and not all_single and device_ids is None:
            shape = self._shape_of(items)
            if shape is not None:
                shape = (klass,) + shape
                if shape in self._shape_graphs:
                    return self._replay_shape(items, self._shape_graphs[shape])
        self._check(items, ahead)
        lens = [len(it.tokens) for it in items]
        b, t = len(items), sum(lens)
        s = sum(len(it.want) for it in items)
        page = self.cache.page_size
        slots_np = np.fromiter((it.slot for it in items), dtype=np.int32, count=b)
        starts_np = np.fromiter((it.start for it in items), dtype=np.int64, count=b)
        ends_np = starts_np + np.asarray(lens, dtype=np.int64)
        self._check_pages(slots_np, starts_np, ends_np)
        capture_shape = False
        if shape is not None:
            self._shapes_seen[shape] = seen = self._shapes_seen.get(shape, 0) + 1
            if len(self._shapes_seen) > 4096:
                self._shapes_seen.clear()
            capture_shape = seen >= self.capture_shapes_from
        static = klass if self.use_graphs and (all_single or capture_shape) else None
        if static is not None:  # the shapes of a captured step may not depend on the step: page tables as wide as the class
            widths = {gi: pages_for(klass, page) for gi in range(len(self.cache.groups))}
        else:
            widths = {gi: pages_for(int(ends_np.max()), page) for gi in range(len(self.cache.groups))}

        lay = _Layout(t, b, s, rows_are_items=static is not None and all_single)
        n_pairs = self.cache.pending_deltas()
        # a captured step keeps room for later steps' pairs: a page per request and what its portions fill
        room = max(n_pairs, 4 * b + 64 + 2 * (t // page)) if static is not None else n_pairs
        total = lay.pairs + 2 * n_pairs
        host = self._staging(total)
        buf = host.numpy()
        views: list[ItemView] = []
        tok = ri = 0
        buf[lay.start] = 0
        for i, (it, n) in enumerate(zip(items, lens)):
            buf[lay.ids + tok: lay.ids + tok + n] = it.tokens
            first = 0 if self.inject_bug == "rope_relative" else it.start
            buf[lay.pos + tok: lay.pos + tok + n] = np.arange(first, first + n, dtype=np.int32)  # absolute positions
            buf[lay.item + tok: lay.item + tok + n] = i
            buf[lay.kvlen + i] = it.start + n - (1 if self.inject_bug == "kv_len_short" and it.start + n > n else 0)
            buf[lay.slot + i] = it.slot
            for w in it.want:
                buf[lay.rows + ri] = tok + w
                buf[lay.rowslot + ri] = it.slot
                ri += 1
            views.append(ItemView(slot=it.slot, start=it.start, end=it.start + n, first_token=tok))
            tok += n
            buf[lay.start + i + 1] = tok
        n_pairs = self.cache.drain_deltas(buf, lay.pairs)

        self.last_h2d_bytes = 4 * total
        if static is not None:
            dev = torch.empty(lay.pairs + 2 * room, dtype=torch.int32, device=self.device)
            dev[:total].copy_(host[:total], non_blocking=True)
        else:
            dev = host[:total].to(self.device, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        if device_ids is not None:
            dev[lay.ids: lay.ids + t].copy_(device_ids)
        rows = dev[lay.rows: lay.rows + s]
        self.last_row_slots = dev[lay.rowslot: lay.rowslot + s]
        with library.pinned_stream():  # one look-up of the stream for the step's hundred-odd launches
            if n_pairs:
                ops.scatter_words(self.cache.resident, dev[lay.pairs:], n_pairs)
            logits = self._device_step(lay, dev, widths, views, lens, static, rows)  # this step's result, computed eagerly
            self.last_tokens = self._choose(logits, self.last_row_slots) if s else None
        self.steps_run += 1
        if static is not None:
            # Capture the same launches for later steps of this batch size and length class.  Nothing runs during capture; the eager
            # run above has already sized every scratch buffer the kernels use.
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before, named = library.launches, library.launch_counts.copy()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                with library.pinned_stream():  # the capture's own stream
                    static_logits = self._device_step(lay, dev, widths, views, lens, static, rows)
                    static_tokens = self._choose(static_logits, self.last_row_slots) if s else None
            recorded = library.launch_counts - named
            made = _DecodeGraph(inputs=dev, logits=static_logits, graph=graph, var_at=lay.var, pairs_at=lay.pairs,
                                pairs_room=room, kernels=library.launches - before, by_name=dict(recorded), layout=lay,
                                tokens=static_tokens)
            if all_single:
                self._graphs[(b, klass)] = made
            else:
                if len(self._shape_graphs) >= self.max_shape_graphs:
                    self._shape_graphs.pop(next(iter(self._shape_graphs)))
                self._shape_graphs[shape] = made
            library.launches = before  # recorded, not run
            library.launch_counts.subtract(recorded)
        return logits

    def _choose(self, logits: torch.Tensor, row_slots: torch.Tensor) -> torch.Tensor | None:
        if not self.sample_in_step:
            return None
        from ..sampling.sampler import choose_tokens
        return choose_tokens(logits, self.cache.records_dev, row_slots)

    def _shape_of(self, items: Sequence[StepItem]) -> tuple | None:
        """What a captured step with prompt portions is keyed by: every item's length and whether it wants the logits
        of its last position (the two forms the scheduler asks for).  None: not a step worth capturing."""
        shape = []
        longest = 0
        for it in items:
            n = len(it.tokens)
            want = tuple(it.want)
            if want == (n - 1,):
                shape.append(n)
            elif want == ():
                shape.append(-n)
            else:
                return None
            longest = max(longest, n)
        if longest > self.longest_captured_portion:
            return None
        return tuple(shape)

    def _replay_shape(self, items: Sequence[StepItem], held: _DecodeGraph) -> torch.Tensor:
        """A step whose shape has been captured: the same checks as the general path, the words that change laid out
        as the capture had them, one copy, one replay."""
        self._check(items)
        cache, lay = self.cache, held.layout
        b = len(items)
        lens = [len(it.tokens) for it in items]
        slots_np = np.fromiter((it.slot for it in items), dtype=np.int32, count=b)
        starts_np = np.fromiter((it.start for it in items), dtype=np.int64, count=b)
        self._check_pages(slots_np, starts_np, starts_np + np.asarray(lens, dtype=np.int64))
        if cache.pending_deltas() > held.pairs_room:
            self._send_deltas_alone()
        n_pairs = cache.pending_deltas()
        words = lay.pairs - lay.var
        total = words + 2 * n_pairs
        host = self._staging(total)
        buf = host.numpy()
        off = -lay.var  # the host buffer starts where the changing words start
        tok = ri = 0
        for i, (it, n) in enumerate(zip(items, lens)):
            buf[off + lay.ids + tok: off + lay.ids + tok + n] = it.tokens
            first = 0 if self.inject_bug == "rope_relative" else it.start
            buf[off + lay.pos + tok: off + lay.pos + tok + n] = np.arange(first, first + n, dtype=np.int32)
            buf[off + lay.kvlen + i] = it.start + n - (1 if self.inject_bug == "kv_len_short" and it.start + n > n else 0)
            buf[off + lay.slot + i] = it.slot
            for _ in it.want:
                buf[off + lay.rowslot + ri] = it.slot
                ri += 1
            tok += n
        n_pairs = cache.drain_deltas(buf, words)
        self.last_h2d_bytes = 4 * total
        held.inputs[lay.var: lay.var + total].copy_(host[:total], non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        self.last_row_slots = held.inputs[lay.rowslot: lay.rowslot + lay.s]
        if n_pairs:
            with library.pinned_stream():
                ops.scatter_words(cache.resident, held.inputs[held.pairs_at:], n_pairs)
        held.graph.replay()
        library.launches += held.kernels
        library.launch_counts.update(held.by_name)
        self.steps_run += 1
        self.graph_replays += 1
        self.last_tokens = held.tokens
        return held.logits

    def _replay(self, items: Sequence[StepItem], held: _DecodeGraph, device_ids: torch.Tensor | None = None,
                ahead: np.ndarray | None = None) -> torch.Tensor:
        """A pure-decode step of a batch size that has been captured: the same checks as the general path, written
        with array operations instead of per-item loops, then one copy of the words that change (token, position,
        length and slot per request, and the resident array's changed words) and one replay."""
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
        self._check_pages(slots, starts, starts + 1)
        if cache.pending_deltas() > held.pairs_room:
            self._send_deltas_alone()
        n_pairs = cache.pending_deltas()
        total = 4 * b + 2 * n_pairs
        host = self._staging(total)
        buf = host.numpy()
        buf[0: b] = toks
        buf[b: 2 * b] = 0 if self.inject_bug == "rope_relative" else starts
        buf[2 * b: 3 * b] = starts + 1 - (1 if self.inject_bug == "kv_len_short" else 0) * (starts > 0)
        buf[3 * b: 4 * b] = slots
        n_pairs = cache.drain_deltas(buf, 4 * b)
        self.last_h2d_bytes = 4 * total
        # ids, positions, lengths and slots are adjacent in the captured buffer and the pairs follow them
        held.inputs[held.var_at: held.var_at + total].copy_(host[:total], non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        if device_ids is not None:
            held.inputs[held.var_at: held.var_at + b].copy_(device_ids)
        self.last_row_slots = held.inputs[held.var_at + 3 * b: held.var_at + 4 * b]
        if n_pairs:
            with library.pinned_stream():
                ops.scatter_words(cache.resident, held.inputs[held.pairs_at:], n_pairs)
        held.graph.replay()
        library.launches += held.kernels  # this library's kernels inside the replayed graph
        library.launch_counts.update(held.by_name)
        self.steps_run += 1
        self.graph_replays += 1
        self.last_tokens = held.tokens
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
