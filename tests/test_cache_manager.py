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
