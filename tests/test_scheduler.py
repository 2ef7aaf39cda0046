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
