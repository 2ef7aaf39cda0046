"""The cache manager: groups, windows, slots; no page lost, held twice or freed twice (CPU)."""

import random

import numpy as np
import pytest
import torch

from prefixserve_b200.cache import CacheError, CacheManager
from prefixserve_b200.parts import CacheNeed, FixedState, PagedKV

FULL = CacheNeed(PagedKV(2, 16))
WINDOWED = CacheNeed(PagedKV(1, 32, window=40))
STATE = CacheNeed(state=FixedState((3, 4)))


def test_groups_follow_the_needs():
    cm = CacheManager([FULL, WINDOWED, FULL, STATE, WINDOWED], num_pages={0: 10, 1: 6}, num_slots=4, max_seq_len=256)
    assert cm.entry_group == [0, 1, 0, None, 1]
    assert [g.window for g in cm.groups] == [None, 40]
    assert cm.num_pages(0) == 10 and cm.num_pages(1) == 6
    assert not cm.prefix_cache_possible and cm.tree is None
    assert CacheManager([FULL, FULL], num_pages=4, num_slots=2, max_seq_len=64).tree is not None
    assert CacheManager([FULL], num_pages=4, num_slots=2, max_seq_len=64, enable_prefix_cache=False).tree is None
    assert CacheManager.bytes_per_page([FULL, WINDOWED, STATE], 16, torch.bfloat16) == 2 * 2 * 16 * 16 * 2 + 2 * 32 * 16 * 2


def test_device_tensors_on_cpu_have_the_documented_layout():
    cm = CacheManager([FULL, STATE], num_pages=5, num_slots=3, max_seq_len=64, page_size=8, dtype=torch.float32, device="cpu")
    assert cm.kv[0].shape == (5, 2, 2, 8, 16) and cm.kv[1] is None
    assert cm.state[1].shape == (3, 3, 4) and cm.state[0] is None
    v = cm.view(0, True)
    assert v.group == 0 and v.page_size == 8 and v.kv is cm.kv[0]
    assert cm.view(1, True).group is None


def test_reserve_is_all_or_nothing_and_pages_come_back():
    cm = CacheManager([FULL, WINDOWED], num_pages={0: 6, 1: 3}, num_slots=2, max_seq_len=128)
    s = cm.open()
    assert cm.reserve(s, 33) and cm.free_pages(0) == 3 and cm.free_pages(1) == 0
    assert not cm.reserve(s, 49)  # the windowed group is short: nothing is taken anywhere
    assert cm.free_pages(0) == 3 and cm.missing(s, 49) == {1: 1}
    cm.advance(s, 48)  # window 40: keys below 9 are out of reach -> page 0 not yet (needs 16 keys gone)
    assert cm.free_pages(1) == 0
    cm.advance(s, 57)  # lowest key 18 -> page 0 is given back
    assert cm.free_pages(1) == 1 and cm.page_ids(s, 1)[0] == -1 and cm.page_ids(s, 0)[0] >= 0
    assert cm.reserve(s, 49)
    cm.check()
    cm.close(s)
    assert cm.free_pages(0) == 6 and cm.free_pages(1) == 3
    with pytest.raises(CacheError, match="not open"):
        cm.close(s)
    cm.check()


def test_limits():
    cm = CacheManager([FULL], num_pages=64, num_slots=1, max_seq_len=40)
    s = cm.open()
    assert cm.open() is None
    with pytest.raises(CacheError, match="max_seq_len"):
        cm.reserve(s, 49)
    assert cm.reserve(s, 40)


def test_fixed_state_is_zeroed_when_a_slot_is_taken():
    cm = CacheManager([STATE], num_pages=1, num_slots=2, max_seq_len=16, device="cpu")
    s = cm.open()
    cm.state[0][s] += 5
    cm.close(s)
    s2 = cm.open()
    assert s2 == s and float(cm.state[0][s2].abs().sum()) == 0


def test_prefix_pages_are_shared_and_counted():
    cm = CacheManager([FULL], num_pages=8, num_slots=3, max_seq_len=128)
    prompt = np.arange(40, dtype=np.int32)
    a = cm.open()
    cm.reserve(a, 40)
    cm.advance(a, 40)
    assert cm.publish(a, prompt) == 2
    matched, pages = cm.match_prefix(prompt[:-1])
    assert matched == 32 and pages == cm.page_ids(a)[:2]
    b = cm.open()
    cm.adopt(b, pages, matched)
    assert cm.position(b) == 32 and cm.reserve(b, 40)
    cm.check()
    cm.close(a)
    assert cm.free_pages() == 8 - 2 - 1 and cm.cached_pages() == 2
    cm.close(b)
    assert cm.evict(5) == 2 and cm.free_pages() == 8
    cm.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_request_orders_lose_nothing(seed):
    """Requests open, grow by random portions, and end in random order; windows release as they go."""
    rng = random.Random(seed)
    cm = CacheManager([FULL, WINDOWED, STATE], num_pages={0: 40, 1: 12}, num_slots=5, max_seq_len=300)
    live: dict[int, int] = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.2 and len(live) < 5:
            s = cm.open()
            assert s is not None and s not in live
            live[s] = 0
        elif r < 0.85 and live:
            s = rng.choice(list(live))
            upto = min(live[s] + rng.choice([1, 1, 2, 7, 16, 33]), 300)
            if cm.reserve(s, upto):
                live[s] = upto
                cm.advance(s, upto)
                held = [p for p in cm.page_ids(s, 1) if p >= 0]
                assert len(held) <= -(-40 // 16) + 2  # a window never holds more than it can reach
        elif live:
            s = rng.choice(list(live))
            cm.close(s)
            del live[s]
        cm.check()
    for s in list(live):
        cm.close(s)
    cm.check()
    assert cm.free_pages(0) == 40 and cm.free_pages(1) == 12 and cm.slots.num_free == 5


@pytest.mark.parametrize("seed", range(4))
def test_changed_words_reach_a_device_copy_through_every_turn_of_a_slot(seed):
    """The page tables and slot records stay on the device; a step sends only the words that changed.  Here the
    "device" is a numpy array that receives nothing but the drained (index, value) pairs, at random moments, while
    slots open, grow, lose pages to their window, close and are reopened.  After every drain the device copy must
    name, for every open slot and every page index a step could read, the page the host holds there."""
    rng = random.Random(seed)
    cm = CacheManager([FULL, WINDOWED], num_pages={0: 30, 1: 10}, num_slots=4, max_seq_len=200)
    device = np.full(cm.resident_words, -1, dtype=np.int32)
    device[: cm.num_slots * cm.record_words] = 0
    live: dict[int, int] = {}
    sampling: dict[int, tuple[float, int]] = {}

    def send():
        n = cm.pending_deltas()
        out = np.zeros(2 * n + 3, dtype=np.int32)
        assert cm.drain_deltas(out, 3) == n and cm.pending_deltas() == 0
        pairs = out[3: 3 + 2 * n].reshape(n, 2)
        assert len(set(pairs[:, 0].tolist())) == n   # every index at most once: the scatter kernel's threads never meet
        device[pairs[:, 0]] = pairs[:, 1]
        for gi, g in enumerate(cm.groups):
            base = cm._table_base[gi]
            rows = device[base: base + cm.num_slots * cm.max_pages_per_seq].reshape(cm.num_slots, cm.max_pages_per_seq)
            for s, upto in live.items():
                first = cm._first_needed_page(g, upto)   # what the next step of this slot can still read
                want = cm.page_ids(s, gi)[first:]
                assert rows[s, first: first + len(want)].tolist() == want and all(p >= 0 for p in want)
        records = device[: cm.num_slots * cm.record_words].reshape(cm.num_slots, cm.record_words)
        for s, (temperature, sd) in sampling.items():
            assert records[s, 1:2].view(np.float32)[0] == np.float32(temperature)
            assert (int(records[s, 2]) & 0xFFFFFFFF) | ((int(records[s, 3]) & 0xFFFFFFFF) << 32) == sd

    for _ in range(400):
        r = rng.random()
        if r < 0.2 and len(live) < 4:
            s = cm.open()
            live[s] = 0
            sampling[s] = (rng.choice([0.0, 0.7, 1.5]), rng.getrandbits(64))
            cm.set_sampling(s, *sampling[s])
        elif r < 0.8 and live:
            s = rng.choice(list(live))
            upto = min(live[s] + rng.choice([1, 1, 3, 16, 40]), 200)
            if cm.reserve(s, upto):
                live[s] = upto
                cm.advance(s, upto)
        elif r < 0.9 and live:   # closed (finished or preempted); the slot comes back to a later request
            s = rng.choice(list(live))
            cm.close(s)
            del live[s], sampling[s]
        if rng.random() < 0.3:
            send()
    send()
    assert cm.pending_deltas() == 0
