"""Host-side launch planning of split-KV decode attention (no GPU needed: pure arithmetic)."""

import random

from prefixserve_b200.ops import tensorcore


def test_key_ranges_cover_the_longest_sequence_in_multiples_of_64():
    rnd = random.Random(0)
    for _ in range(2000):
        pairs = rnd.randint(1, 2048)
        longest = rnd.randint(1, 20000)
        sms = rnd.choice([1, 16, 132, 148])
        chunk = tensorcore._decode_key_range(pairs, longest, sms, rnd.random() < 0.5)
        assert chunk >= 64 and chunk % 64 == 0
        assert -(-longest // chunk) * chunk >= longest
        assert chunk >= min(tensorcore.MIN_KEY_RANGE, -(-longest // 64) * 64) or chunk >= longest


def test_one_round_of_the_shortest_ranges_that_fit():
    slots = tensorcore.DECODE_CTAS_PER_SM * 148
    for pairs, longest in ((8, 4096), (64, 4096), (128, 4096), (256, 4096), (64, 8192)):
        chunk = tensorcore._decode_key_range(pairs, longest, 148, False)  # (one kernel for every range: no step at 1,024)
        ranges = -(-longest // chunk)
        assert pairs * ranges <= slots                      # one round
        if chunk > tensorcore.MIN_KEY_RANGE:                # and no shorter range would still make one round
            shorter = -(-(-(-longest // (ranges + 1))) // 64) * 64
            assert shorter == chunk or pairs * -(-longest // shorter) > slots


def test_several_rounds_where_one_would_leave_many_slots_empty():
    # 48 requests, 8 key/value heads, 4,096 keys: 384 whole sequences fill two thirds of the 592 slots; thirds of them
    # make two rounds of a third the length each (measured: 2.00 against 2.34 ms a decode step)
    assert tensorcore._decode_key_range(48 * 8, 4096, 148, True) == 1408
    # 64 requests fill 512 of 592 slots: nothing shorter pays
    assert tensorcore._decode_key_range(64 * 8, 4096, 148, True) == 4096
    # heads of 128: an SM holds two CTAs, so eight requests take four ranges of 1,024 keys, not eight of 512
    assert tensorcore._decode_key_range(8 * 8, 4096, 148, True, 2) == 1024
    assert tensorcore._decode_key_range(8 * 8, 4096, 148, True, 4) == 512


def test_length_classes_of_captured_steps():
    from prefixserve_b200.engine.step import ModelRunner
    assert ModelRunner._length_classes(8192) == (1024, 2048, 4096, 8192)
    assert ModelRunner._length_classes(256) == (256,)            # shorter than the smallest class: one class
    assert ModelRunner._length_classes(1024) == (1024,)
    assert ModelRunner._length_classes(5000) == (1024, 2048, 4096, 5000)
    assert ModelRunner._length_classes(300, 64) == (64, 128, 256, 300)


def test_the_few_row_kernels_reduction_covers_every_row_once():
    """csrc/kernels/gemm_tcgen05_fewrows.cu: after the cluster barrier, CTA `rank` of `ks` adds up the partial sums of rows
    rank, rank + ks, ... : thread e (0..127) takes row rank + ks * (e >> 5) and every 4 * ks-th after it, four features
    wide (plain products; a warp a row), or rank + ks * (e >> 4) and every 8 * ks-th with sixteen threads a row (gated).
    In front of a norm a thread fetches the stream's pieces of its first EARLY rows before the accumulator is complete
    and picks them by it = (row - rank) / ks / 4.  Restated here: every (row, feature) is taken exactly once, and the
    early pieces are the ones used."""
    early = 4
    for ks in (1, 2, 4, 8):
        for m in range(1, 65):
            plain, gated = {}, {}
            for rank in range(ks):
                for e in range(128):
                    rows = list(range(rank + ks * (e >> 5), m, 4 * ks))
                    for it, t in enumerate(rows):
                        for f in range((e & 31) * 4, (e & 31) * 4 + 4):
                            plain[(t, f)] = plain.get((t, f), 0) + 1
                        assert (t - rank) // ks // 4 == it
                        if it < early:  # fetched ahead as row rank + ks * ((e >> 5) + 4 * it)
                            assert rank + ks * ((e >> 5) + 4 * it) == t
                    for t in range(rank + ks * (e >> 4), m, 8 * ks):
                        for f in range((e & 15) * 4, (e & 15) * 4 + 4):   # gate features f.., up features 64 + f..
                            gated[(t, f)] = gated.get((t, f), 0) + 1
            assert plain == {(t, f): 1 for t in range(m) for f in range(128)}, (ks, m)
            assert gated == {(t, f): 1 for t in range(m) for f in range(64)}, (ks, m)
