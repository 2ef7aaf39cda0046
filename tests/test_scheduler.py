"""The scheduler's decisions, with a fake sampler and no device (CPU).

The rules checked are those PrefixServe pins in tests/test_scheduler.py: decodes
run every step and cost no budget, prompts are cut into portions under a shared
budget, a shared prompt is reused, an identical prompt still computes a token,
running out of pages preempts the newest and never the oldest, a preempted
request finds its own pages again, aborts in flight are deferred, refusals,
finishing on length and on stop ids, and the schedule/commit protocol.
"""

import numpy as np
import pytest

from prefixserve_b200.engine import AddResult, FinishReason, Scheduler, SchedulerError
from prefixserve_b200.engine.scheduler import host_only_cache


def drive(s, budget=512, seqs=64, token=lambda rid, n: 1000 + n, max_steps=10_000, on_batch=None):
    """Runs to completion; returns request id -> generated tokens and the list of batches."""
    out, batches = {}, []
    for _ in range(max_steps):
        if not s.has_work():
            break
        batch = s.schedule_step(budget, seqs)
        batches.append([(w.req.req_id, w.start, w.end) for w in batch.work])
        if on_batch:
            on_batch(batch)
        sampled = {w.req.req_id: token(w.req.req_id, len(w.req.output)) for w in batch.work if w.samples}
        res = s.commit(batch, sampled)
        for rid, tok in res.new_tokens.items():
            out.setdefault(rid, []).append(tok)
        s.cache.check()
    assert not s.has_work()
    return out, batches


def prompt(n, base=0):
    return np.arange(base, base + n, dtype=np.int32)


def test_decodes_run_every_step_and_ignore_the_budget():
    s = Scheduler(64, chunk_size=512)
    for i in range(3):
        assert s.add_request(f"r{i}", prompt(5, 100 * i), 4) is AddResult.ACCEPTED
    out, batches = drive(s, budget=5)  # the budget only admits one prompt per step
    assert [len(b) for b in batches[:3]] == [1, 2, 3]
    assert batches[1][0] == ("r0", 5, 6)  # r0 decodes while r1 is admitted
    assert all(len(v) == 4 for v in out.values())


def test_long_prompt_is_cut_into_portions():
    s = Scheduler(128, chunk_size=512)
    s.add_request("a", prompt(1300), 1)
    _, batches = drive(s)
    assert batches == [[("a", 0, 512)], [("a", 512, 1024)], [("a", 1024, 1300)]]


def test_budget_is_shared_between_prompts():
    s = Scheduler(128, chunk_size=512)
    s.add_request("a", prompt(600), 1)
    s.add_request("b", prompt(300, 5000), 1)
    _, batches = drive(s, budget=600)
    assert batches[0] == [("a", 0, 512), ("b", 0, 88)]
    assert batches[1] == [("a", 512, 600), ("b", 88, 300)]


def test_shared_prompt_is_reused_after_it_completed():
    s = Scheduler(128)
    system = list(range(256))
    s.add_request("a", system + [900, 901], 2)
    drive(s)
    s.add_request("b", system + [800, 801, 802], 2)
    batch = s.schedule_step(512, 8)
    assert [(w.start, w.end) for w in batch.work] == [(256, 259)]
    assert s.get_request("b").cached_tokens == 256
    s.commit(batch, {"b": 1})
    assert s.stats().cached_prompt_tokens == 256 and s.stats().prefix_hit_rate == 256 / (258 + 259)


def test_identical_prompt_still_computes_a_token():
    s = Scheduler(64)
    s.add_request("a", prompt(64), 1)
    drive(s)
    s.add_request("b", prompt(64), 1)
    batch = s.schedule_step(512, 8)
    assert [(w.start, w.end, w.samples) for w in batch.work] == [(48, 64, True)]
    s.commit(batch, {"b": 3})


def test_requests_admitted_in_one_step_do_not_share():
    s = Scheduler(64)
    s.add_request("a", prompt(40), 1)
    s.add_request("b", prompt(40), 1)
    batch = s.schedule_step(512, 8)
    assert [(w.start, w.end) for w in batch.work] == [(0, 40), (0, 40)]
    s.commit(batch, {"a": 1, "b": 1})


def test_out_of_pages_preempts_the_newest_never_the_oldest():
    s = Scheduler(6, chunk_size=512)  # 96 tokens of cache
    s.add_request("old", prompt(30), 40, ignore_eos=True)
    s.add_request("new", prompt(30, 500), 40, ignore_eos=True)
    preempted = []
    out, _ = drive(s, on_batch=lambda b: preempted.extend(b.preempted))
    assert preempted and set(preempted) == {"new"}
    assert len(out["old"]) == 40 and len(out["new"]) == 40  # outputs survive preemption
    assert s.stats().preemptions == len(preempted)
    assert s.stats().free_blocks + s.stats().cached_blocks == 6


def test_preempted_request_finds_its_pages_again():
    s = Scheduler(8)
    s.add_request("old", prompt(60), 50, ignore_eos=True)
    s.add_request("new", prompt(40, 500), 30, ignore_eos=True)
    seen = {}

    def watch(batch):
        for w in batch.work:
            if w.req.req_id == "new" and w.req.num_preemptions and "back" not in seen:
                seen["back"] = (w.start, w.req.cached_tokens)

    drive(s, on_batch=watch)
    assert "back" in seen and seen["back"][0] >= 16  # re-admission starts after the pages of its own that survived


def test_admission_never_preempts_and_keeps_arrival_order():
    s = Scheduler(4)
    s.add_request("a", prompt(40), 20, ignore_eos=True)
    b1 = s.schedule_step(512, 8)
    s.commit(b1, {"a": 1})
    s.add_request("big", prompt(33, 900), 1)   # needs 3 pages, one is free
    s.add_request("small", prompt(3, 700), 1)  # would fit, but must not overtake
    b2 = s.schedule_step(512, 8)
    assert [w.req.req_id for w in b2.work] == ["a"] and b2.preempted == []
    s.commit(b2, {"a": 1})


def test_running_cap():
    s = Scheduler(64)
    for i in range(5):
        s.add_request(f"r{i}", prompt(4, 50 * i), 3)
    batch = s.schedule_step(512, 2)
    assert len(batch.work) == 2 and s.stats().num_waiting == 3
    s.commit(batch, {w.req.req_id: 1 for w in batch.work})


def test_finish_on_length_and_on_stop_ids():
    s = Scheduler(16, stop_token_ids=[7, 9])
    s.add_request("len", prompt(3), 2)
    s.add_request("stop", prompt(3, 50), 10)
    s.add_request("deaf", prompt(3, 90), 3, ignore_eos=True)
    finished = {}
    while s.has_work():
        b = s.schedule_step(512, 8)
        res = s.commit(b, {w.req.req_id: (5 if w.req.req_id == "len" else 9) for w in b.work if w.samples})
        finished.update(res.finished)
    assert finished == {"stop": FinishReason.STOP, "len": FinishReason.LENGTH, "deaf": FinishReason.LENGTH}


def test_finished_prompt_stays_cached():
    s = Scheduler(16)
    s.add_request("a", prompt(40), 1)
    drive(s)
    st = s.stats()
    assert st.cached_blocks == 2 and st.free_blocks == 14 and st.num_running == 0


def test_prefix_cache_switch():
    s = Scheduler(16, enable_prefix_cache=False)
    s.add_request("a", prompt(40), 1)
    drive(s)
    s.add_request("b", prompt(40), 1)
    b = s.schedule_step(512, 8)
    assert [(w.start, w.end) for w in b.work] == [(0, 40)] and s.stats().cached_blocks == 0
    s.commit(b, {"b": 1})


def test_abort_waiting_running_and_in_flight():
    s = Scheduler(16)
    s.add_request("w", prompt(5), 5)
    assert s.free_request("w") and not s.free_request("w") and not s.free_request("nobody")
    s.add_request("a", prompt(20), 5)
    s.add_request("b", prompt(20, 100), 5)
    batch = s.schedule_step(512, 8)
    assert s.free_request("a")          # in flight: deferred
    assert s.get_request("a") is not None and not s.free_request("a")
    res = s.commit(batch, {"a": 1, "b": 1})
    assert res.finished == {"a": FinishReason.ABORT} and s.get_request("a") is None
    assert s.free_request("b")          # nothing in flight: immediate
    assert not s.has_work()
    s.cache.check()
    assert s.stats().free_blocks + s.stats().cached_blocks == 16


def test_refusals():
    s = Scheduler(4, max_waiting=2)
    assert s.add_request("", [1], 1) is AddResult.INVALID
    assert s.add_request("x", [], 1) is AddResult.INVALID
    assert s.add_request("x", [1.5], 1) is AddResult.INVALID
    assert s.add_request("x", [[1, 2]], 1) is AddResult.INVALID
    assert s.add_request("x", [-1], 1) is AddResult.INVALID
    assert s.add_request("x", [2**31], 1) is AddResult.INVALID
    assert s.add_request("x", [1], 0) is AddResult.INVALID
    assert s.add_request("x", [1], True) is AddResult.INVALID
    assert s.add_request("x", prompt(60), 5) is AddResult.TOO_LONG  # 65 tokens > 4 pages
    assert s.add_request("x", prompt(60), 4) is AddResult.ACCEPTED
    assert s.add_request("x", [1], 1) is AddResult.DUPLICATE_ID
    assert s.add_request("y", [1], 1) is AddResult.ACCEPTED
    assert s.add_request("z", [1], 1) is AddResult.QUEUE_FULL
    assert s.stats().rejected == 11


def test_prompt_is_copied():
    s = Scheduler(8)
    mine = np.arange(5, dtype=np.int64)
    s.add_request("a", mine, 1)
    mine[:] = 0
    assert s.get_request("a").prompt.tolist() == [0, 1, 2, 3, 4] and s.get_request("a").prompt.dtype == np.int32


def test_protocol_errors():
    s = Scheduler(8)
    s.add_request("a", prompt(3), 2)
    with pytest.raises(ValueError):
        s.schedule_step(0, 1)
    with pytest.raises(ValueError):
        s.schedule_step(1, 0)
    batch = s.schedule_step(512, 8)
    with pytest.raises(SchedulerError, match="committed"):
        s.schedule_step(512, 8)
    with pytest.raises(SchedulerError, match="no token"):
        s.commit(batch, {})
    s2 = Scheduler(8)
    s2.add_request("a", prompt(3), 2)
    other = s2.schedule_step(512, 8)
    with pytest.raises(SchedulerError, match="not the one in flight"):
        s.commit(other, {"a": 1})
    with pytest.raises(ValueError):
        Scheduler(8, chunk_size=0)


def test_request_tokens_slices():
    s = Scheduler(8)
    s.add_request("a", prompt(5), 9)
    r = s.get_request("a")
    r.output.extend([50, 51, 52])
    full = r.seq().tolist()
    for lo in range(8):
        for hi in range(lo + 1, 9):
            assert r.tokens(lo, hi).tolist() == full[lo:hi]


def test_windowed_model_frees_pages_as_it_decodes():
    """With a windowed group beside a full one, commit() releases what the window has passed."""
    from prefixserve_b200.cache import CacheManager
    from prefixserve_b200.parts import CacheNeed, PagedKV
    cache = CacheManager([CacheNeed(PagedKV(1, 8)), CacheNeed(PagedKV(1, 8, window=20))], num_pages={0: 16, 1: 4},
                         num_slots=4, max_seq_len=256)
    s = Scheduler(cache, chunk_size=16)
    assert not s._share_prefixes
    s.add_request("a", prompt(30), 100, ignore_eos=True)
    out, _ = drive(s)
    assert len(out["a"]) == 100 and cache.free_pages(1) == 4 and cache.free_pages(0) == 16


def test_cache_given_or_made():
    cache = host_only_cache(12, page_size=8)
    s = Scheduler(cache, chunk_size=8)
    s.add_request("a", prompt(20), 3)
    _, batches = drive(s)
    assert batches[:3] == [[("a", 0, 8)], [("a", 8, 16)], [("a", 16, 20)]]
    assert s.stats().cached_blocks == 2  # pages of 8 tokens


# ---- scheduling one step ahead of the commit ------------------------------------------------------------------------

def drive_ahead(s, budget=512, seqs=64, token=lambda rid, n: 1000 + n):
    """The loop of the entry point with a fake device: a step is 'launched' when it is scheduled and its tokens are
    only made up when it is finished, after the next step has been scheduled ahead if that was possible."""
    out, kinds = {}, []
    pending = None
    while pending is not None or s.has_work():
        if pending is None:
            pending = s.schedule_step(budget, seqs)
            kinds.append("plain")
        ahead = s.schedule_ahead(seqs)
        if ahead is not None:
            kinds.append("ahead")
            assert [w.req for w in ahead.work] == [w.req for w in pending.work if w.samples]
            assert all(w.ahead and w.samples and w.end - w.start == 1 for w in ahead.work)
        counts = {w.req.req_id: len(w.req.output) for w in pending.work}
        sampled = {w.req.req_id: token(w.req.req_id, counts[w.req.req_id]) for w in pending.work
                   if w.samples and w.req.req_id in s._by_id}
        res = s.commit(pending, sampled)
        for rid, tok in res.new_tokens.items():
            out.setdefault(rid, []).append(tok)
        s.cache.check()
        pending = ahead
    return out, kinds


def test_ahead_gives_the_same_tokens_and_is_used_for_plain_decoding():
    def build():
        s = Scheduler(64, stop_token_ids=[1003])
        s.add_request("a", prompt(20), 9, ignore_eos=True)
        s.add_request("b", prompt(7, 100), 30)            # stops at its fourth token (1003), found out one step late
        s.add_request("c", prompt(40, 200), 6, ignore_eos=True)
        return s
    plain, _ = drive(build())
    ahead, kinds = drive_ahead(build())
    assert ahead == plain
    assert plain["b"] == [1000, 1001, 1002, 1003] and len(plain["a"]) == 9 and len(plain["c"]) == 6
    assert kinds.count("ahead") >= 4 and kinds[0] == "plain"


def test_ahead_is_refused_where_the_next_step_depends_on_this_one():
    s = Scheduler(16)
    assert s.schedule_ahead() is None                       # nothing in flight
    s.add_request("a", prompt(40), 3, ignore_eos=True)
    b = s.schedule_step(16, 4)                              # a prompt portion that samples nothing
    assert s.schedule_ahead() is None
    s.commit(b, {})
    b = s.schedule_step(16, 4)
    s.commit(b, {})
    b = s.schedule_step(16, 4)                              # the last portion: samples token 1 of 3
    assert [w.samples for w in b.work] == [True]
    nxt = s.schedule_ahead()
    assert nxt is not None and [(w.start, w.end) for w in nxt.work] == [(40, 41)]
    assert s.schedule_ahead() is None                       # only one step ahead
    with pytest.raises(SchedulerError):
        s.schedule_step(16, 4)
    s.commit(b, {"a": 5})
    last = s.schedule_ahead()                               # the step in flight yields token 2 of 3, this one the third
    assert last is not None and [(w.start, w.end) for w in last.work] == [(41, 42)]
    with pytest.raises(SchedulerError):
        s.commit(b, {"a": 5})
    res = s.commit(nxt, {"a": 6})
    assert res.new_tokens == {"a": 6} and not res.finished
    assert s.schedule_ahead() is None                       # nothing follows the last token
    res = s.commit(last, {"a": 7})
    assert res.finished == {"a": FinishReason.LENGTH} and not s.has_work()
    # someone waiting who could be admitted, an abort, and a lack of pages all send the caller the ordinary way
    s = Scheduler(8)
    assert s.add_request("x", prompt(30), 50, ignore_eos=True) is AddResult.ACCEPTED
    b = s.schedule_step(64, 1)
    s.add_request("y", prompt(3), 5)
    assert s.schedule_ahead(2) is None and s.schedule_ahead() is None
    assert s.schedule_ahead(1) is not None                  # y cannot be admitted anyway: x holds the only seat
    s = Scheduler(4, enable_prefix_cache=False)
    for rid in ("x", "y"):
        assert s.add_request(rid, prompt(31), 20, ignore_eos=True) is AddResult.ACCEPTED
    b = s.schedule_step(64, 2)                              # 31 tokens each: two pages each, the pool is used up
    nxt = s.schedule_ahead()
    assert nxt is not None                                  # position 31 still lies in the second page
    s.commit(b, {"x": 1, "y": 1})
    assert s.schedule_ahead() is None                       # position 32 needs a third page: someone has to go, which
    s.commit(nxt, {"x": 2, "y": 2})                         # only the ordinary way decides
    b = s.schedule_step(64, 2)
    assert b.preempted == ["y"] and [w.req.req_id for w in b.work] == ["x"]
    s.commit(b, {"x": 3})
    s = Scheduler(16)
    s.add_request("x", prompt(5), 50, ignore_eos=True)
    b = s.schedule_step(64, 1)
    s.free_request("x")
    assert s.schedule_ahead() is None
    assert s.commit(b, {"x": 1}).finished == {"x": FinishReason.ABORT}


def test_abort_while_two_steps_are_out():
    s = Scheduler(16)
    s.add_request("x", prompt(5), 50, ignore_eos=True)
    s.add_request("y", prompt(6, 50), 50, ignore_eos=True)
    b = s.schedule_step(64, 4)
    nxt = s.schedule_ahead()
    assert nxt is not None
    assert s.free_request("x")                              # both steps may still write into its pages
    res = s.commit(b, {"x": 1, "y": 2})
    assert res.finished == {"x": FinishReason.ABORT}
    res = s.commit(nxt, {"x": 3, "y": 4})                   # what the step ahead computed for x is dropped
    assert res.new_tokens == {"y": 4} and not res.finished
    s.cache.check()
    assert s.stats().num_running == 1


# ---- later additions -------------------------------------------------------------------------------------------------

def test_a_request_may_bring_stop_ids_of_its_own():
    from prefixserve_b200 import SamplingParams
    s = Scheduler(64, chunk_size=512, stop_token_ids=[1003])
    s.add_request("own", prompt(5), 10, sampling=SamplingParams(max_tokens=10, stop_token_ids=(1001,)))
    s.add_request("model", prompt(5, 50), 10)
    s.add_request("deaf", prompt(5, 90), 6, ignore_eos=True, sampling=SamplingParams(max_tokens=6, stop_token_ids=(1001,)))
    out, _ = drive(s)
    assert out["own"] == [1000, 1001]                 # its own id ends it, the id itself is kept
    assert out["model"] == [1000, 1001, 1002, 1003]   # the model's id still applies to the others
    assert len(out["deaf"]) == 6


def test_a_windowed_pool_too_small_for_one_portion_is_refused_at_the_door():
    """A group with a window holds the window, the portion being computed and one page of slack; a request that could
    never hold that is refused when it is added instead of being preempted by itself for ever."""
    from prefixserve_b200.cache import CacheManager
    from prefixserve_b200.parts import CacheNeed, PagedKV
    needs = [CacheNeed(PagedKV(1, 8)), CacheNeed(PagedKV(1, 8, window=20))]
    small = CacheManager(needs, num_pages={0: 64, 1: 3}, num_slots=4, max_seq_len=512)
    s = Scheduler(small, chunk_size=32)   # window 20 + portion 32 = 52 tokens = 4 pages, + 1 of slack
    assert s.add_request("long", prompt(200), 20) is AddResult.TOO_LONG
    assert s.add_request("short", prompt(30), 10) is AddResult.ACCEPTED   # 40 tokens never need more than 3 pages
    enough = CacheManager(needs, num_pages={0: 64, 1: 5}, num_slots=4, max_seq_len=512)
    s = Scheduler(enough, chunk_size=32)
    assert s.add_request("long", prompt(200), 20, ignore_eos=True) is AddResult.ACCEPTED
    out, _ = drive(s)
    assert len(out["long"]) == 20 and s.stats().preemptions == 0


def test_a_failed_step_leaves_nothing_behind():
    """The entry point's loop with an engine that fails once: the call raises, every request of the call is gone,
    slots and pages are back, and the next call works."""
    from prefixserve_b200 import SamplingParams
    from prefixserve_b200.engine.llm import LLM

    class Pending:
        def __init__(self, batch):
            self.batch = batch

    class FlakyEngine:
        def __init__(self):
            self.fail_at, self.launched = 3, 0

        def launch(self, batch, feed=None):
            self.launched += 1
            if self.launched == self.fail_at:
                raise RuntimeError("device fault")
            return Pending(batch)

        def finish(self, pending):
            return {w.req.req_id: 7 for w in pending.batch.work if w.samples}

        def check_device_status(self):
            pass

    llm = LLM.__new__(LLM)
    llm.engine = FlakyEngine()
    llm.scheduler = Scheduler(host_only_cache(32, num_slots=4), chunk_size=16)
    llm.max_running_requests, llm.chunked_prefill_size, llm._counter = 4, 16, 0
    params = SamplingParams(max_tokens=5, ignore_eos=True)
    with pytest.raises(RuntimeError, match="device fault"):
        llm.generate([list(range(20)), list(range(40, 50))], params)
    s = llm.scheduler
    assert not s.has_work() and s._inflight is None and s._ahead is None
    s.cache.check()
    assert s.cache.slots.num_free == 4 and s.cache.free_pages(0) + s.cache.cached_pages() == 32
    assert llm.generate([list(range(20))], params) == [[7] * 5]   # the next call starts clean
