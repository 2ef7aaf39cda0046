"""The cache manager: pages of keys and values, page tables, request slots.

Every cache entry of a model (one per writing mixer call) states a need:
keys and values for all tokens, for a window of them, and/or a fixed-size
state per request.  Entries whose paged need has the same window form a
*group*; a group has a page pool of its own (ids, reference counts), one page
table row per request slot, and its entries' tensors are indexed by the same
page id.  A request holds one slot; the slot indexes the page table rows and
the fixed-state tensors.

Pages are taken when a step needs them, given back when the request ends, is
preempted, or (window groups) when the window has passed them, and reused.
Finished prompts can be kept in a prefix tree for other requests
(one group of full attention only; anything with a window or a carried state
cannot restore from a prefix, so the tree is off for such models).

The reference keeps this split between a C++ pool/tree and Python lists on the
request (csrc/block_manager.hpp, csrc/radix_tree.hpp,
prefixserve/scheduler.py:370-451, prefixserve/llama_engine.py:110-117); here
one object owns ids, tables, slots and the device tensors.
Cache layout of an entry: [num_pages, 2 (key, value), kv_heads, page_size, head_dim].

What a step needs to know about a request stays on the device in one int32
array (``resident``): a record per slot (position, sampling temperature and
seed) followed by every group's page table rows [num_slots, max_pages].  The
C++ side holds the mirror and logs which words changed; ``drain_deltas`` hands
a step the (index, value) pairs to send, and nothing else of the tables
travels.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Sequence

import numpy as np
import torch

from ..parts.base import CacheNeed, CacheView
from .core import BlockManager, CoreError, RadixTree, SeqTables, SlotPool, SlotRecords


class CacheError(RuntimeError):
    pass


def pages_for(tokens: int, page_size: int) -> int:
    return -(-tokens // page_size)


@dataclass
class _Group:
    window: int | None
    pool: BlockManager
    tables: SeqTables
    entries: list[int]


class CacheManager:
    def __init__(
        self,
        needs: Sequence[CacheNeed],
        *,
        num_pages: int | Mapping[int, int],
        num_slots: int,
        max_seq_len: int,
        page_size: int = 16,
        dtype: torch.dtype = torch.bfloat16,
        device: torch.device | str | None = None,
        enable_prefix_cache: bool = True,
        hash_seed: int | None = None,
    ) -> None:
        if page_size < 1 or num_slots < 1 or max_seq_len < 1:
            raise ValueError("page_size, num_slots and max_seq_len must be >= 1")
        self.page_size = page_size
        self.num_slots = num_slots
        self.max_seq_len = max_seq_len
        self.max_pages_per_seq = pages_for(max_seq_len, page_size)
        self.needs = list(needs)
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None

        # group entries by window
        self.groups: list[_Group] = []
        self.entry_group: list[int | None] = []
        by_window: dict[int | None, int] = {}
        for i, need in enumerate(self.needs):
            if need.paged is None:
                self.entry_group.append(None)
                continue
            w = need.paged.window
            if w is not None and w < 1:
                raise ValueError(f"cache entry {i}: window {w} must be >= 1")
            if w not in by_window:
                by_window[w] = len(self.groups)
                n = num_pages[len(self.groups)] if isinstance(num_pages, Mapping) else int(num_pages)
                self.groups.append(_Group(w, BlockManager(n), SeqTables(num_slots, self.max_pages_per_seq), []))
            g = by_window[w]
            self.groups[g].entries.append(i)
            self.entry_group.append(g)

        # Test hook: fill every page with NaN the moment nobody holds it any more, so that a step which still reads a
        # page it has given back (or reads a reused page beyond what its new owner wrote) cannot go unnoticed.
        self.poison_freed = False
        self.slots = SlotPool(num_slots)
        self.records = SlotRecords(num_slots)          # host mirror of the per-slot records, owned by the C++ side
        self._position = self.records.view()[:, 0]     # tokens computed, per slot (a view of the mirror)
        self.record_words = SlotRecords.WORDS
        # where each mirrored array starts in the device's resident array
        self._table_base: list[int] = []
        at = num_slots * self.record_words
        for _ in self.groups:
            self._table_base.append(at)
            at += num_slots * self.max_pages_per_seq
        self.resident_words = at

        has_state = any(n.state is not None for n in self.needs)
        self.prefix_cache_possible = len(self.groups) == 1 and self.groups[0].window is None and not has_state
        self.tree: RadixTree | None = None
        if enable_prefix_cache and self.prefix_cache_possible:
            self.tree = RadixTree(self.groups[0].pool, page_size, hash_seed)

        # device tensors
        self.kv: list[torch.Tensor | None] = [None] * len(self.needs)
        self.state: list[torch.Tensor | None] = [None] * len(self.needs)
        self._pools: list = []  # the kernel library's allocations behind ``kv``
        self.resident: torch.Tensor | None = None
        self.records_dev: torch.Tensor | None = None
        self.tables_dev: list[torch.Tensor] = []
        if self.device is not None:
            self.resident = torch.full((self.resident_words,), -1, dtype=torch.int32, device=self.device)
            self.records_dev = self.resident[: num_slots * self.record_words].view(num_slots, self.record_words)
            self.records_dev.zero_()
            self.tables_dev = [self.resident[b: b + num_slots * self.max_pages_per_seq].view(num_slots, self.max_pages_per_seq)
                               for b in self._table_base]
            for i, need in enumerate(self.needs):
                if need.paged is not None:
                    g = self.groups[self.entry_group[i]]
                    shape = (g.pool.num_blocks, 2, need.paged.num_kv_heads, page_size, need.paged.head_dim)
                    self.kv[i] = self._pages(shape, dtype)
                if need.state is not None:
                    self.state[i] = torch.zeros((num_slots, *need.state.shape), dtype=need.state.dtype, device=self.device)

    def _pages(self, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        """The pages of one cache entry, zeroed.  On a CUDA device the memory belongs to the kernel library's pool
        (allocated once, at a fixed address, freed with this manager); elsewhere (bookkeeping tests on the host) it is
        an ordinary tensor."""
        if self.device.type != "cuda":
            return torch.zeros(shape, dtype=dtype, device=self.device)
        from ..ops.library import DevicePool
        count = 1
        for n in shape:
            count *= int(n)
        pool = DevicePool(count * torch.empty((), dtype=dtype).element_size(), self.device)
        self._pools.append(pool)
        return pool.tensor(shape, dtype)

    def release_device_memory(self) -> None:
        """Gives the pages' device memory back now (waits for the device).  The manager is of no use afterwards."""
        self.kv = [None] * len(self.needs)
        for pool in self._pools:
            pool.free()
        self._pools.clear()

    # ------------------------------------------------------------------ sizes
    @staticmethod
    def bytes_per_page(needs: Sequence[CacheNeed], page_size: int, dtype: torch.dtype) -> int:
        """Bytes one page id costs over all entries (all groups counted as one, for sizing a single-group model)."""
        return sum(CacheManager.group_page_bytes(needs, page_size, dtype).values())

    @staticmethod
    def group_page_bytes(needs: Sequence[CacheNeed], page_size: int, dtype: torch.dtype) -> dict[int | None, int]:
        """window (None: all keys) -> bytes one page id of that group costs over the group's entries, in the order
        in which the groups are numbered (first appearance among the entries)."""
        item = torch.empty((), dtype=dtype).element_size()
        out: dict[int | None, int] = {}
        for n in needs:
            if n.paged is not None:
                out[n.paged.window] = out.get(n.paged.window, 0) + 2 * n.paged.num_kv_heads * page_size * n.paged.head_dim * item
        return out

    def num_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_blocks

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def cached_pages(self) -> int:
        return self.tree.num_cached_blocks if self.tree is not None else 0

    # ------------------------------------------------------------------ slots
    def open(self) -> int | None:
        """A slot for a new request, its fixed states zeroed; None when all are taken."""
        slot = self.slots.take()
        if slot is None:
            return None
        self._position[slot] = 0
        for st in self.state:
            if st is not None:
                st[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        """Gives back every page the slot holds, then the slot."""
        if not self.slots.taken(slot):
            raise CacheError(f"slot {slot} is not open (closed twice?)")
        for g in self.groups:
            ids = g.tables.clear(slot)
            try:
                g.pool.decref_many(ids)
            except CoreError as e:  # a page freed twice: never continue silently
                raise CacheError(f"slot {slot}: {e}") from e
            self._poison(g, ids)
        self._position[slot] = 0
        self.slots.give_back(slot)

    def _poison(self, g: _Group, ids: Sequence[int]) -> None:
        if not self.poison_freed or not ids:
            return
        free = [p for p in ids if g.pool.ref_count(p) == 0]
        if free:
            index = torch.tensor(free, device=self.device)
            for entry in g.entries:
                if self.kv[entry] is not None:
                    self.kv[entry][index] = float("nan")

    def position(self, slot: int) -> int:
        return int(self._position[slot])

    def set_sampling(self, slot: int, temperature: float, seed: int) -> None:
        """Notes how the slot's request samples; the sampling kernel reads it from the slot's record on the device."""
        self.records.set_sampling(slot, float(temperature), int(seed) & 0xFFFFFFFFFFFFFFFF)

    # ----------------------------------------------------- what the device holds
    def pending_deltas(self) -> int:
        """Words of the resident array (records, page tables) that changed since the device last saw them."""
        return self.records.pending + sum(g.tables.pending for g in self.groups)

    def drain_deltas(self, out: np.ndarray, at: int) -> int:
        """Writes the changed words as (index into ``resident``, value) pairs into the int32 array ``out`` from word
        ``at`` on (2 * pending_deltas() words) and forgets them.  Returns the number of pairs."""
        n = self.records.drain(0, out, at)
        for base, g in zip(self._table_base, self.groups):
            n += g.tables.drain(base, out, at + 2 * n)
        return n

    def covered(self, group: int, slots: np.ndarray, first: np.ndarray, upto: np.ndarray) -> int:
        """Index of the first of ``slots`` whose row in ``group`` lacks a valid page at some page index in
        [first, upto); -1 when every row is whole."""
        g = self.groups[group]
        return int(g.tables.covered(slots, first, upto, g.pool.num_blocks))

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, g: _Group, upto_start: int) -> int:
        """Lowest page index a query at position >= upto_start can still read."""
        if g.window is None:
            return 0
        lowest_key = max(0, upto_start - g.window + 1)
        return lowest_key // self.page_size

    def shortfall(self, slot: int, upto: int) -> dict[int, int]:
        """Pages still to take, per group, so that positions < upto are covered. {} when nothing is missing."""
        need: dict[int, int] = {}
        want = pages_for(upto, self.page_size)
        if want > self.max_pages_per_seq:
            raise CacheError(f"{upto} tokens exceed the engine's max_seq_len {self.max_seq_len}")
        for gi, g in enumerate(self.groups):
            more = want - g.tables.length(slot)
            if more > 0:
                need[gi] = more
        return need

    def reserve(self, slot: int, upto: int) -> bool:
        """Takes the pages needed to hold positions < upto. All or nothing; False when a pool is short."""
        need = self.shortfall(slot, upto)
        for gi, n in need.items():
            if self.groups[gi].pool.num_free < n:
                return False
        for gi, n in need.items():
            g = self.groups[gi]
            ids = g.pool.allocate_many(n)
            assert ids is not None
            g.tables.append(slot, ids)
        return True

    def missing(self, slot: int, upto: int) -> dict[int, int]:
        """Per group, how many pages a reserve(slot, upto) would lack right now."""
        return {gi: n - self.groups[gi].pool.num_free for gi, n in self.shortfall(slot, upto).items()
                if self.groups[gi].pool.num_free < n}

    def adopt(self, slot: int, page_ids: Sequence[int], tokens: int) -> None:
        """Starts a fresh slot with pages matched in the prefix tree (the caller already holds their references)."""
        if len(self.groups) != 1:
            raise CacheError("prefix pages can only be adopted by a single-group cache")
        g = self.groups[0]
        if g.tables.length(slot) != 0:
            raise CacheError(f"slot {slot} already holds pages")
        g.tables.append(slot, list(page_ids))
        self._position[slot] = tokens

    def advance(self, slot: int, computed: int) -> None:
        """Records that positions < computed are in the cache; window groups give back pages now out of reach."""
        self._position[slot] = computed
        for g in self.groups:
            if g.window is None:
                continue
            ids = g.tables.release_front(slot, self._first_needed_page(g, computed))
            if ids:
                g.pool.decref_many(ids)
                self._poison(g, ids)

    def page_ids(self, slot: int, group: int = 0) -> list[int]:
        return self.groups[group].tables.row(slot)

    def tables_for(self, slots: Sequence[int], widths: Mapping[int, int] | None = None) -> dict[int, np.ndarray]:
        """group -> int32 [len(slots), width] page ids by absolute page index (-1 where nothing is held)."""
        out: dict[int, np.ndarray] = {}
        arr = np.asarray(slots, dtype=np.int32)
        for gi, g in enumerate(self.groups):
            width = (widths or {}).get(gi) or max([g.tables.length(s) for s in slots] + [1])
            dense = np.empty((len(slots), width), dtype=np.int32)
            g.tables.gather(arr, width, dense)
            out[gi] = dense
        return out

    # ------------------------------------------------------------ prefix tree
    def match_prefix(self, tokens: np.ndarray) -> tuple[int, list[int]]:
        if self.tree is None:
            return 0, []
        return self.tree.match_prefix(tokens)

    def publish(self, slot: int, tokens: np.ndarray) -> int:
        """Puts the slot's full pages covering ``tokens`` into the prefix tree. Returns pages added."""
        if self.tree is None or len(tokens) < self.page_size:
            return 0
        return self.tree.insert(tokens, self.groups[0].tables.row(slot))

    def release_pages(self, page_ids: Sequence[int], group: int = 0) -> None:
        self.groups[group].pool.decref_many(list(page_ids))

    def evict(self, pages: int) -> int:
        if self.tree is None or pages <= 0:
            return 0
        return self.tree.evict(pages)

    def is_cached(self, page_id: int) -> bool:
        return self.tree is not None and self.tree.is_cached(page_id)

    # ------------------------------------------------------------------ views
    def view(self, entry: int, writes: bool) -> CacheView:
        return CacheView(group=self.entry_group[entry], kv=self.kv[entry], state=self.state[entry],
                         page_size=self.page_size, writes=writes)

    # ------------------------------------------------------------- invariants
    def check(self) -> None:
        """No page lost, held twice by mistake, or freed twice: counts must equal holders."""
        for gi, g in enumerate(self.groups):
            g.pool.check_invariants()
            holders = np.zeros(g.pool.num_blocks, dtype=np.int64)
            for s in range(self.num_slots):
                row = g.tables.row(s)
                if row and not self.slots.taken(s):
                    raise CacheError(f"group {gi}: closed slot {s} still holds pages")
                for p in row:
                    if p >= 0:
                        holders[p] += 1
            if self.tree is not None and gi == 0:
                self.tree.check_invariants()
                for p in range(g.pool.num_blocks):
                    if self.tree.is_cached(p):
                        holders[p] += 1
            for p in range(g.pool.num_blocks):
                rc = g.pool.ref_count(p)
                if rc != holders[p]:
                    raise CacheError(f"group {gi}: page {p} has count {rc} but {holders[p]} holders")
            free = int((holders == 0).sum())
            if free != g.pool.num_free:
                raise CacheError(f"group {gi}: {g.pool.num_free} pages free, {free} unheld")
