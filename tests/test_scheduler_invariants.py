"""Random sequences of add / abort / step against a small pool: nothing leaks, everything finishes (CPU)."""

import numpy as np
from hypothesis import settings, strategies as st
from hypothesis.stateful import RuleBasedStateMachine, invariant, precondition, rule

from prefixserve_b200.engine import AddResult, Scheduler

POOL = 24


class Machine(RuleBasedStateMachine):
    def __init__(self):
        super().__init__()
        self.s = Scheduler(POOL, chunk_size=24, max_waiting=16, stop_token_ids=[3])
        self.n = 0
        self.produced: dict[str, int] = {}

    @rule(length=st.integers(1, 120), max_tokens=st.integers(1, 40), shared=st.booleans(), deaf=st.booleans())
    def add(self, length, max_tokens, shared, deaf):
        base = 0 if shared else 1000 * (self.n + 1)
        rid = f"r{self.n}"
        self.n += 1
        verdict = self.s.add_request(rid, np.arange(base, base + length) % 50000, max_tokens, ignore_eos=deaf)
        assert verdict in (AddResult.ACCEPTED, AddResult.TOO_LONG, AddResult.QUEUE_FULL)
        if verdict is AddResult.ACCEPTED:
            self.produced[rid] = 0

    @rule(which=st.integers(0, 200))
    def abort(self, which):
        self.s.free_request(f"r{which}")

    @rule(budget=st.integers(1, 64), seqs=st.integers(1, 6), tok=st.integers(0, 9), abort_mid=st.booleans())
    def step(self, budget, seqs, tok, abort_mid):
        batch = self.s.schedule_step(budget, seqs)
        ids = [w.req.req_id for w in batch.work]
        assert len(ids) == len(set(ids))
        for w in batch.work:
            assert 0 <= w.start < w.end <= w.req.seq_len
            assert len(self.s.block_table(w.req)) * 16 >= w.end
        assert sum(w.end - w.start for w in batch.work if w.end - w.start > 1) <= budget
        if abort_mid and batch.work:
            self.s.free_request(batch.work[0].req.req_id)
        res = self.s.commit(batch, {w.req.req_id: tok for w in batch.work if w.samples})
        for rid in res.new_tokens:
            self.produced[rid] += 1

    @invariant()
    def nothing_leaks(self):
        self.s.cache.check()
        st_ = self.s.stats()
        held = set()
        for rid in list(self.produced):
            req = self.s.get_request(rid)
            if req is not None and req.slot is not None:
                held.update(self.s.block_table(req))
        assert st_.free_blocks + len(held | {p for p in range(POOL) if self.s.cache.is_cached(p)}) == POOL

    def teardown(self):
        # everything left finishes without further input
        for _ in range(5000):
            if not self.s.has_work():
                break
            batch = self.s.schedule_step(32, 4)
            self.s.commit(batch, {w.req.req_id: 1 for w in batch.work if w.samples})
        assert not self.s.has_work()
        self.s.cache.check()
        st_ = self.s.stats()
        assert st_.free_blocks + st_.cached_blocks == POOL


TestSchedulerMachine = Machine.TestCase
TestSchedulerMachine.settings = settings(max_examples=60, stateful_step_count=40, deadline=None)
