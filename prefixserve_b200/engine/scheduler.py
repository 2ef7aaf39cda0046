"""Continuous batching: who runs in the next step, with how many tokens.

Rules, after the reference's scheduler (prefixserve/scheduler.py:143-451):

* A request is its token list (prompt + generated) and a count of tokens whose
  keys and values are in the cache.  A step gives it the next portion of the
  uncomputed tail; when the portion reaches the end of the list a token is
  sampled.  One token left = decode; more = prefill; after a preemption the
  same path recomputes.
* Running requests are served oldest first.  Decodes always run and cost no
  budget; portions of prompts share ``max_prefill_tokens`` per step and are at
  most ``chunk_size`` long; a prompt whose budget is used up waits a step.
* Waiting requests are admitted first-come-first-served while fewer than
  ``max_decode_seqs`` run.  Admission matches the longest cached prefix of all
  but the last token, takes pages for the first portion only, may evict cached
  pages but never preempts; if the head of the queue cannot start, nobody
  behind it does.
* When a running request needs pages and none are free: evict unused cached
  pages; if that is not enough, preempt the newest running request (its full
  pages go to the prefix cache, its count returns to zero, it goes to the
  front of the queue) and try again.  The asker may preempt itself.  The
  oldest request can always take from newer ones, and add_request refuses
  anything that could not fit alone, so the oldest always finishes.
* schedule_step and commit alternate; aborts of running requests that arrive
  in between take effect at commit.
"""

from __future__ import annotations

import bisect
import logging
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Iterable, Mapping

import numpy as np

from ..cache.manager import CacheManager, pages_for
from ..parts.base import CacheNeed, PagedKV
from ..sampling import SamplingParams

log = logging.getLogger(__name__)

DEFAULT_CHUNK_SIZE = 512
SLOW_STEP_SECONDS = 1e-3


class SchedulerError(RuntimeError):
    """schedule_step/commit were called out of order, or with the wrong batch."""


class ReqState(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(str, Enum):
    LENGTH = "length"
    STOP = "stop"
    ABORT = "abort"


class AddResult(Enum):
    ACCEPTED = "accepted"
    QUEUE_FULL = "queue_full"
    TOO_LONG = "too_long"
    DUPLICATE_ID = "duplicate_id"
    INVALID = "invalid"


@dataclass(eq=False)
class Request:
    req_id: str
    prompt: np.ndarray
    max_tokens: int
    arrival: int
    ignore_eos: bool = False
    sampling: SamplingParams = field(default_factory=SamplingParams)
    state: ReqState = ReqState.WAITING
    output: list[int] = field(default_factory=list)
    slot: int | None = None
    num_computed: int = 0
    cached_tokens: int = 0
    num_preemptions: int = 0
    abort_pending: bool = False
    prompt_cached: bool = False

    @property
    def seq_len(self) -> int:
        return len(self.prompt) + len(self.output)

    def seq(self) -> np.ndarray:
        if not self.output:
            return self.prompt
        return np.concatenate((self.prompt, np.asarray(self.output, dtype=np.int32)))

    def tokens(self, start: int, end: int) -> np.ndarray:
        """seq()[start:end] without building the whole list."""
        n = len(self.prompt)
        if end <= n:
            return self.prompt[start:end]
        tail = np.asarray(self.output[max(start - n, 0): end - n], dtype=np.int32)
        return tail if start >= n else np.concatenate((self.prompt[start:], tail))


@dataclass(frozen=True)
class WorkItem:
    req: Request
    start: int
    end: int
    ahead: bool = False  # scheduled before the step in front of it was committed: its one token is not known yet

    @property
    def samples(self) -> bool:
        return self.ahead or self.end == self.req.seq_len


@dataclass(frozen=True)
class Batch:
    work: list[WorkItem]
    preempted: list[str]

    @property
    def num_tokens(self) -> int:
        return sum(w.end - w.start for w in self.work)


@dataclass(frozen=True)
class StepResult:
    new_tokens: dict[str, int]
    finished: dict[str, FinishReason]


@dataclass(frozen=True)
class SchedulerStats:
    num_waiting: int
    num_running: int
    free_blocks: int
    cached_blocks: int
    prompt_tokens: int
    cached_prompt_tokens: int
    preemptions: int
    rejected: int

    @property
    def prefix_hit_rate(self) -> float:
        return self.cached_prompt_tokens / self.prompt_tokens if self.prompt_tokens else 0.0


def host_only_cache(num_blocks: int, *, page_size: int = 16, num_slots: int = 256, enable_prefix_cache: bool = True,
                    max_seq_len: int | None = None) -> CacheManager:
    """Bookkeeping without device tensors: one group of full attention (scheduler tests, simulations)."""
    need = CacheNeed(paged=PagedKV(num_kv_heads=1, head_dim=1))
    return CacheManager([need], num_pages=num_blocks, num_slots=num_slots,
                        max_seq_len=max_seq_len or num_blocks * page_size, page_size=page_size, device=None,
                        enable_prefix_cache=enable_prefix_cache)


class _StepPlan:
    """What schedule_step is putting together: the work so far, who was preempted for it, the prompt tokens left."""

    def __init__(self, budget: int) -> None:
        self.work: list[WorkItem] = []
        self.preempted: list[str] = []
        self.budget = budget

    def take(self, item: WorkItem, is_prompt: bool) -> None:
        if is_prompt:  # single decoded tokens are free; portions of prompts (and recomputation) pay
            self.budget -= item.end - item.start
        self.work.append(item)


class Scheduler:
    def __init__(
        self,
        cache: CacheManager | int,
        *,
        max_waiting: int = 1024,
        chunk_size: int = DEFAULT_CHUNK_SIZE,
        stop_token_ids: Iterable[int] = (),
        enable_prefix_cache: bool = True,
    ) -> None:
        if max_waiting < 1 or chunk_size < 1:
            raise ValueError("max_waiting and chunk_size must be >= 1")
        if isinstance(cache, int):
            cache = host_only_cache(cache, enable_prefix_cache=enable_prefix_cache)
        self.cache = cache
        self._share_prefixes = enable_prefix_cache and cache.tree is not None
        self._max_waiting = max_waiting
        self._chunk = chunk_size
        self._stop = frozenset(int(t) for t in stop_token_ids)

        self._by_id: dict[str, Request] = {}
        self._waiting: deque[Request] = deque()
        self._running: list[Request] = []  # by arrival, newest last
        self._inflight: Batch | None = None
        self._ahead: Batch | None = None  # scheduled after _inflight, before its commit (schedule_ahead)
        self._abort_at_commit: list[Request] = []
        self._arrivals = 0
        self._n_prompt = self._n_prompt_cached = self._n_preempt = self._n_rejected = 0

    # ------------------------------------------------------------ interface
    def add_request(self, req_id: str, prompt, max_tokens: int, *, ignore_eos: bool = False,
                    sampling: SamplingParams | None = None) -> AddResult:
        verdict, tokens = self._vet(req_id, prompt, max_tokens)
        if verdict is not AddResult.ACCEPTED:
            self._n_rejected += 1
            return verdict
        req = Request(req_id, tokens, max_tokens, self._arrivals, ignore_eos, sampling or SamplingParams())
        self._arrivals += 1
        self._by_id[req_id] = req
        self._waiting.append(req)
        self._n_prompt += len(tokens)
        return verdict

    def schedule_step(self, max_prefill_tokens: int, max_decode_seqs: int) -> Batch:
        if self._inflight is not None:
            raise SchedulerError("the previous batch has not been committed")
        if max_prefill_tokens < 1 or max_decode_seqs < 1:
            raise ValueError("max_prefill_tokens and max_decode_seqs must be >= 1")  # 0 would stall prompts forever
        t0 = time.perf_counter()
        plan = _StepPlan(max_prefill_tokens)
        self._plan_running(plan)
        self._plan_admissions(plan, max_decode_seqs)
        batch = Batch(plan.work, plan.preempted)
        self._inflight, self._ahead = batch, None
        took = time.perf_counter() - t0
        if took > SLOW_STEP_SECONDS:
            log.debug("schedule_step took %.2f ms", took * 1e3)
        return batch

    def schedule_ahead(self, max_decode_seqs: int | None = None) -> Batch | None:
        """The step after the one in flight, decided before that one's tokens are known, so that the device need not
        wait for the host between two decode steps.

        Possible when every request of the batch in flight gets a token from it and goes on afterwards whatever that
        token is, except that it may be a stop token: then the request's share of the step ahead is thrown away at its
        commit.  Returns None whenever the ordinary way is needed instead: a request reaches its length limit, an abort
        is pending, someone waits and could be admitted (``max_decode_seqs`` as for schedule_step; None: anyone waiting
        counts), or pages would have to be taken from another request.
        """
        cur = self._inflight
        if cur is None or self._ahead is not None or not cur.work or self._abort_at_commit:
            return None
        if self._waiting and (max_decode_seqs is None or len(self._running) < max_decode_seqs):
            return None
        for w in cur.work:
            req = w.req
            if req.state is not ReqState.RUNNING:
                return None  # it ended with the step before: the step in flight carries it for nothing, the next must not
            if not w.samples or req.abort_pending or len(req.output) + 1 >= req.max_tokens or w.end + 1 > self.cache.max_seq_len:
                return None
        work = []
        for w in cur.work:
            if not self._take_pages(w.req, w.end + 1):
                return None  # pages taken for the requests before this one stay theirs: they need them next step anyway
            work.append(WorkItem(w.req, w.end, w.end + 1, ahead=True))
        self._ahead = Batch(work, [])
        return self._ahead

    def commit(self, batch: Batch, sampled: Mapping[str, int]) -> StepResult:
        if batch is not self._inflight:
            raise SchedulerError("commit() was given a batch that is not the one in flight")
        self._inflight, self._ahead = self._ahead, None  # a step scheduled ahead is the one in flight from now on
        new_tokens: dict[str, int] = {}
        finished: dict[str, FinishReason] = {}
        for w in batch.work:
            req = w.req
            if w.ahead and req.state is not ReqState.RUNNING:
                continue  # it ended with the step before (a stop token): what this step computed for it is dropped
            if req.num_computed != w.start:
                raise SchedulerError(f"{req.req_id}: the batch is stale")
            sampling = w.samples  # asked before the count moves: it compares the item's end with the sequence length
            req.num_computed = w.end
            self.cache.advance(req.slot, w.end)
            if not sampling:
                continue
            try:
                token = int(sampled[req.req_id])
            except KeyError:
                raise SchedulerError(f"no token was returned for {req.req_id}") from None
            new_tokens[req.req_id] = token
            reason = self._take_token(req, token)
            if reason is not None:
                self._retire(req)
                finished[req.req_id] = reason
        for req in self._abort_at_commit:  # aborts that had to wait because the batch could still write their pages
            if req.state is ReqState.RUNNING:
                self._retire(req)
                finished[req.req_id] = FinishReason.ABORT
        self._abort_at_commit.clear()
        return StepResult(new_tokens, finished)

    def abandon_inflight(self) -> None:
        """After a step failed on the device: forgets the batch in flight (and one scheduled ahead) without a commit.
        Requests keep what their last commit recorded; aborts that waited for the commit take effect now."""
        self._inflight = self._ahead = None
        for req in self._abort_at_commit:
            if req.state is ReqState.RUNNING:
                self._retire(req)
        self._abort_at_commit.clear()

    def free_request(self, req_id: str) -> bool:
        """Aborts a request; harmless for unknown ids and when called twice."""
        req = self._by_id.get(req_id)
        if req is None or req.abort_pending:
            return False
        if req.state is ReqState.RUNNING and self._inflight is not None:
            req.abort_pending = True  # the batch in flight may still write into its pages: ended at the commit
            self._abort_at_commit.append(req)
        elif req.state is ReqState.RUNNING:
            self._retire(req)
        else:  # waiting: it holds nothing
            self._waiting.remove(req)
            req.state = ReqState.FINISHED
            del self._by_id[req_id]
        return True

    def get_request(self, req_id: str) -> Request | None:
        return self._by_id.get(req_id)

    def has_work(self) -> bool:
        return bool(self._waiting) or bool(self._running)

    def block_table(self, req: Request) -> list[int]:
        return self.cache.page_ids(req.slot) if req.slot is not None else []

    def stats(self) -> SchedulerStats:
        return SchedulerStats(
            num_waiting=len(self._waiting),
            num_running=len(self._running),
            free_blocks=self.cache.free_pages(0),
            cached_blocks=self.cache.cached_pages(),
            prompt_tokens=self._n_prompt,
            cached_prompt_tokens=self._n_prompt_cached,
            preemptions=self._n_preempt,
            rejected=self._n_rejected,
        )

    # ------------------------------------------------------------ one step
    def _portion(self, remaining: int, budget: int) -> int:
        """How many of a request's uncomputed tokens run now: its one decoded token whatever the budget says,
        otherwise as much of the tail as the portion limit and the step's budget allow (0: it waits a step)."""
        return 1 if remaining == 1 else min(self._chunk, remaining, budget)

    def _plan_running(self, plan: _StepPlan) -> None:
        """The requests that already run, oldest first.  One that needs pages takes them from the newest running
        request; a victim is always newer than the asker, so it has no work in the plan yet."""
        for req in list(self._running):
            if req.state is not ReqState.RUNNING:
                continue  # preempted a moment ago for an older request
            remaining = req.seq_len - req.num_computed
            n = self._portion(remaining, plan.budget)
            if n and self._secure(req, req.num_computed + n, plan.preempted):
                plan.take(WorkItem(req, req.num_computed, req.num_computed + n), is_prompt=remaining > 1)

    def _plan_admissions(self, plan: _StepPlan, max_running: int) -> None:
        """Newcomers in order of arrival, while there is room to run them; the first that cannot start holds up the rest."""
        while self._waiting and len(self._running) < max_running:
            item = self._start(self._waiting[0], plan.budget)
            if item is None:
                return
            self._waiting.popleft()
            plan.take(item, is_prompt=item.end - item.start > 1)

    def _take_token(self, req: Request, token: int) -> FinishReason | None:
        """Appends a sampled token; says why the request ends with it, if it does."""
        if not req.prompt_cached:  # prompt complete for the first time: others may share it from now on
            self._publish(req)
            req.prompt_cached = True
        req.output.append(token)
        if req.abort_pending:
            return None  # ended below, with the other deferred aborts
        stops = not req.ignore_eos and (token in self._stop or token in req.sampling.stop_token_ids)
        if stops:
            return FinishReason.STOP  # the stop token itself is kept
        return FinishReason.LENGTH if len(req.output) >= req.max_tokens else None

    # ------------------------------------------------------------ admission control
    def _vet(self, req_id, prompt, max_tokens) -> tuple[AddResult, np.ndarray | None]:
        """(verdict, the prompt as an int32 array of our own).  A request is refused if it is malformed, if its id is
        in use, if it could not fit even alone (too many positions, or more pages than a group has: every page in a
        group that keeps all keys; the window, a portion and a page of slack in one that keeps a window), or if the
        queue is full.  The checks run in that order and the first that fails names the verdict."""
        arr = None
        if isinstance(req_id, str) and req_id and type(max_tokens) is int and max_tokens >= 1:
            try:
                arr = np.asarray(prompt)
            except (TypeError, ValueError, OverflowError):
                arr = None
        well_formed = (arr is not None and arr.ndim == 1 and arr.size > 0 and arr.dtype.kind in "iu"
                       and int(arr.min()) >= 0 and int(arr.max()) <= np.iinfo(np.int32).max)
        if not well_formed:
            return AddResult.INVALID, None
        total = int(arr.size) + max_tokens
        page = self.cache.page_size

        def most_pages(g) -> int:
            whole = pages_for(total, page)
            return whole if g.window is None else min(whole, pages_for(g.window + self._chunk, page) + 1)

        checks = (
            (req_id in self._by_id, AddResult.DUPLICATE_ID),
            (total > self.cache.max_seq_len or any(most_pages(g) > g.pool.num_blocks for g in self.cache.groups), AddResult.TOO_LONG),
            (len(self._waiting) >= self._max_waiting, AddResult.QUEUE_FULL),
        )
        for failed, verdict in checks:
            if failed:
                return verdict, None
        return AddResult.ACCEPTED, arr.astype(np.int32)  # a copy: later changes by the caller do not reach us

    # ------------------------------------------------------------ pages
    def _take_pages(self, req: Request, upto: int) -> bool:
        """reserve, evicting unused cached pages if that is what it takes."""
        if self.cache.reserve(req.slot, upto):
            return True
        lacking = self.cache.missing(req.slot, upto)
        if set(lacking) != {0} or self.cache.tree is None:
            return False
        self.cache.evict(lacking[0])
        return self.cache.reserve(req.slot, upto)

    def _secure(self, req: Request, upto: int, preempted: list[str]) -> bool:
        """Pages for a running request, taken from the newest running one for as long as that is what it takes.
        False: the request ended up preempting itself."""
        while not self._take_pages(req, upto):
            victim = self._running[-1]
            self._preempt(victim)
            preempted.append(victim.req_id)
            if victim is req:
                return False
        return True

    def _start(self, req: Request, budget: int) -> WorkItem | None:
        """Admits the head of the queue with its first portion, or leaves everything as it was."""
        seq = req.seq()
        # all but the last token may come from the prefix cache: the last one's logits are what the request is after
        matched, pages = self.cache.match_prefix(seq[:-1]) if self._share_prefixes else (0, [])
        n = self._portion(len(seq) - matched, budget)
        slot = self.cache.open() if n > 0 else None
        if slot is None:
            self.cache.release_pages(pages)
            return None
        req.slot = slot
        self.cache.set_sampling(slot, req.sampling.temperature, req.sampling.seed)
        if pages:
            self.cache.adopt(slot, pages, matched)
        if not self._take_pages(req, matched + n):
            self.cache.close(slot)  # returns the matched pages too; admission never preempts
            req.slot = None
            return None
        req.num_computed = matched
        req.cached_tokens += matched
        if req.num_preemptions == 0:
            self._n_prompt_cached += min(matched, len(req.prompt))
        req.state = ReqState.RUNNING
        bisect.insort(self._running, req, key=lambda r: r.arrival)
        return WorkItem(req, matched, matched + n)

    def _publish(self, req: Request) -> None:
        if self._share_prefixes and req.num_computed >= self.cache.page_size:
            self.cache.publish(req.slot, req.seq()[: req.num_computed])

    def _leave_running(self, req: Request) -> None:
        """What ending and preempting share: full pages to the prefix tree, slot and pages back."""
        self._publish(req)
        self.cache.close(req.slot)
        req.slot = None
        self._running.remove(req)

    def _preempt(self, req: Request) -> None:
        """Recomputation, not swapping: the request starts over at the front of the queue; what it had computed
        stays findable in the prefix cache."""
        self._leave_running(req)
        req.num_computed = 0
        req.num_preemptions += 1
        req.state = ReqState.WAITING
        self._waiting.appendleft(req)
        self._n_preempt += 1

    def _retire(self, req: Request) -> None:
        self._leave_running(req)
        req.state = ReqState.FINISHED
        del self._by_id[req.req_id]
