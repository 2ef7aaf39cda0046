"""The host C++ module: page pool, prefix tree, slots, page tables (CPU).

Cases follow the behaviour PrefixServe pins in tests/cpp/test_core.cpp and
tests/test_core_bindings.py (allocation order, last-in-first-out reuse, double
free refused, whole pages only, siblings that start alike, atomic insert,
least-recently-used eviction that skips pages in use and walks up a chain, a
randomised model check of the reference counts).
"""

import random

import numpy as np
import pytest

from prefixserve_b200.cache import BLOCK_SIZE, BlockManager, CoreError, RadixTree, SeqTables, SlotPool


def toks(*blocks, tail=0):
    out = []
    for b in blocks:
        out += [b * 1000 + i for i in range(16)]
    return np.asarray(out + [7] * tail, dtype=np.int32)


def test_block_size_and_pool_limits():
    assert BLOCK_SIZE == 16
    for bad in (0, -1, (1 << 26) + 1):
        with pytest.raises(ValueError):
            BlockManager(bad)


def test_allocation_order_and_reuse():
    bm = BlockManager(4)
    assert [bm.allocate() for _ in range(4)] == [0, 1, 2, 3]
    assert bm.allocate() is None and bm.num_free == 0
    bm.decref(1)
    bm.decref(3)
    assert bm.allocate() == 3 and bm.allocate() == 1  # last freed comes back first
    bm.check_invariants()


def test_reference_counts_and_double_free():
    bm = BlockManager(2)
    a = bm.allocate()
    bm.incref(a)
    assert bm.ref_count(a) == 2
    bm.decref(a)
    assert bm.num_free == 1
    bm.decref(a)
    assert bm.num_free == 2 and bm.ref_count(a) == 0
    with pytest.raises(CoreError, match="double free"):
        bm.decref(a)
    with pytest.raises(CoreError, match="double free"):
        bm.incref(a)
    assert bm.num_free == 2  # the refused call changed nothing
    for bad in (-1, 2):
        with pytest.raises(CoreError, match="out of range"):
            bm.ref_count(bad)
        with pytest.raises(CoreError, match="out of range"):
            bm.decref(bad)
    bm.check_invariants()


def test_allocate_many_is_all_or_nothing():
    bm = BlockManager(5)
    assert bm.allocate_many(3) == [0, 1, 2]
    assert bm.allocate_many(3) is None and bm.num_free == 2
    assert bm.allocate_many(0) == []
    with pytest.raises(ValueError):
        bm.allocate_many(-1)
    ids = bm.allocate_many(2)
    ids.append(99)  # the returned list is a copy
    assert bm.num_free == 0
    with pytest.raises(CoreError, match="index 2"):
        bm.decref_many([0, 1, 1, 2])
    assert bm.ref_count(0) == 0 and bm.ref_count(1) == 0 and bm.ref_count(2) == 1
    bm.decref_many(np.asarray([2, 3], dtype=np.int64))
    with pytest.raises(ValueError):
        bm.decref_many(np.zeros((2, 2), dtype=np.int32))


def test_tree_matches_whole_pages_only():
    bm = BlockManager(8)
    tree = RadixTree(bm, 16, 1)
    assert tree.match_prefix(toks(1, 2)) == (0, [])
    ids = bm.allocate_many(3)
    assert tree.insert(toks(1, 2, tail=9), ids) == 2  # the partial page is not cached
    assert tree.num_cached_blocks == 2 and not tree.is_cached(ids[2])
    assert tree.match_prefix(toks(1, 2, 3)) == (32, ids[:2])
    assert tree.match_prefix(toks(1, tail=15)) == (16, ids[:1])
    assert tree.match_prefix(toks(2, 1)) == (0, [])
    assert bm.ref_count(ids[0]) == 1 + 1 + 2  # holder, tree, two matches
    tree.check_invariants()


def test_siblings_and_depth():
    bm = BlockManager(8)
    tree = RadixTree(bm, 16, 2)
    a = toks(1)
    b = a.copy()
    b[15] += 1  # same start, different end: a different child
    ia, ib = bm.allocate_many(2)
    tree.insert(a, [ia])
    tree.insert(b, [ib])
    assert tree.match_prefix(a) == (16, [ia]) and tree.match_prefix(b) == (16, [ib])
    # the same tokens one level down are another node
    ic = bm.allocate()
    tree.insert(np.concatenate([a, a]), [ia, ic])
    assert tree.match_prefix(np.concatenate([a, a]))[1] == [ia, ic]
    assert tree.num_cached_blocks == 3
    tree.check_invariants()


def test_duplicate_content_keeps_the_trees_copy():
    bm = BlockManager(8)
    tree = RadixTree(bm, 16, 3)
    first = bm.allocate_many(2)
    tree.insert(toks(1, 2), first)
    mine = bm.allocate_many(3)
    assert tree.insert(toks(1, 2, 3), mine) == 1  # only the third page is adopted
    assert tree.match_prefix(toks(1, 2, 3))[1] == first + [mine[2]]
    assert not tree.is_cached(mine[0]) and tree.is_cached(mine[2])


def test_insert_is_atomic():
    bm = BlockManager(8)
    tree = RadixTree(bm, 16, 4)
    ids = bm.allocate_many(3)
    cached = bm.allocate()
    tree.insert(toks(9), [cached])
    free_one = bm.allocate()
    bm.decref(free_one)
    for bad, word in (([ids[0], 99, ids[2]], "out of range"), ([ids[0], free_one, ids[2]], "not allocated"),
                      ([ids[0], cached, ids[2]], "already owned"), ([ids[0], ids[1], ids[0]], "already owned")):
        with pytest.raises(CoreError, match=word):
            tree.insert(toks(1, 2, 3), bad)
        assert tree.num_cached_blocks == 1 and not tree.is_cached(ids[0])
        tree.check_invariants()
    with pytest.raises(ValueError):
        tree.insert(toks(1, 2, 3), ids[:2])  # fewer ids than full pages
    assert tree.insert(toks(1, 2, 3), ids) == 3


def test_eviction_order_in_use_and_chains():
    bm = BlockManager(8)
    tree = RadixTree(bm, 16, 5)
    a, b, c = bm.allocate_many(1), bm.allocate_many(1), bm.allocate_many(3)
    tree.insert(toks(1), a)
    tree.insert(toks(2), b)
    tree.insert(toks(3, 4, 5), c)
    bm.decref_many(a + c)            # b is still held by a request
    tree.match_prefix(toks(1))       # touch a: now newer than the chain... and take a reference
    bm.decref(a[0])
    assert tree.evict(1) == 1 and not tree.is_cached(c[2]) and tree.is_cached(c[1])  # deepest of the oldest chain
    assert tree.evict(10) == 3       # rest of the chain, then a; b is skipped because it is in use
    assert tree.is_cached(b[0]) and tree.num_cached_blocks == 1
    bm.decref(b[0])
    assert tree.evict(1) == 1 and bm.num_free == 8
    tree.check_invariants()
    bm.check_invariants()


def test_tree_gives_references_back_and_keeps_pool_alive():
    bm = BlockManager(4)
    tree = RadixTree(bm, 16, 6)
    ids = bm.allocate_many(2)
    tree.insert(toks(1, 2), ids)
    bm.decref_many(ids)
    assert bm.num_free == 2
    del tree
    assert bm.num_free == 4
    tree2 = RadixTree(BlockManager(2))  # the pool stays alive through the tree
    assert tree2.match_prefix(toks(1)) == (0, [])


def test_other_page_lengths():
    bm = BlockManager(8)
    tree = RadixTree(bm, 5, 7)
    ids = bm.allocate_many(3)
    t = np.arange(13, dtype=np.int32)
    assert tree.insert(t, ids) == 2 and tree.block_size == 5
    assert tree.match_prefix(t[:11]) == (10, ids[:2])


def test_randomised_reference_counts():
    rng = random.Random(0)
    bm = BlockManager(24)
    tree = RadixTree(bm, 16, 8)
    holders: list[list[int]] = []
    vocab_blocks = 6
    for _ in range(4000):
        op = rng.random()
        if op < 0.35:
            n = rng.randint(1, 4)
            seq = toks(*[rng.randrange(vocab_blocks) for _ in range(n)])
            matched, got = tree.match_prefix(seq)
            need = n - len(got)
            new = bm.allocate_many(need)
            if new is None:
                tree.evict(need - bm.num_free)
                new = bm.allocate_many(need)
            if new is None:
                bm.decref_many(got)
                continue
            table = got + new
            tree.insert(seq, table)
            holders.append(table)
        elif op < 0.8 and holders:
            bm.decref_many(holders.pop(rng.randrange(len(holders))))
        else:
            tree.evict(rng.randint(1, 3))
        cached = sum(tree.is_cached(p) for p in range(24))
        assert cached == tree.num_cached_blocks
        for p in range(24):
            assert bm.ref_count(p) == tree.is_cached(p) + sum(t.count(p) for t in holders)
    tree.check_invariants()
    bm.check_invariants()
    for t in holders:
        bm.decref_many(t)
    tree.evict(24)
    assert bm.num_free == 24


def test_slots_and_page_tables():
    pool = SlotPool(2)
    a, b = pool.take(), pool.take()
    assert (a, b) == (0, 1) and pool.take() is None
    pool.give_back(a)
    with pytest.raises(CoreError, match="twice"):
        pool.give_back(a)
    assert pool.taken(b) and not pool.taken(a) and pool.num_free == 1

    tables = SeqTables(3, 5)
    tables.append(1, [7, 8, 9])
    tables.append(1, [4])
    assert tables.row(1) == [7, 8, 9, 4] and tables.length(1) == 4 and tables.length(0) == 0
    assert tables.release_front(1, 2) == [7, 8] and tables.first_live(1) == 2
    assert tables.row(1) == [-1, -1, 9, 4]
    assert tables.release_front(1, 1) == []  # already gone
    out = np.zeros((2, 6), dtype=np.int32)
    tables.gather([1, 0], 6, out)
    assert out.tolist() == [[-1, -1, 9, 4, -1, -1], [-1] * 6]
    with pytest.raises(CoreError, match="full"):
        tables.append(1, [1, 2])
    assert tables.clear(1) == [9, 4] and tables.length(1) == 0
    with pytest.raises(ValueError):
        tables.append(3, [1])
