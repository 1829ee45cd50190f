"""The rule by which the fused GEMM + reduce-scatter publishes a finished tile, restated on the CPU.

Four epilogue warps each store 32 rows of every tile and keep one monotonic counter each (tiles stored so
far).  The warps are not in lock step: with two accumulator buffers a warp can be up to two tiles ahead of
the slowest one.  A tile may be announced to its owner only when all four warps have stored it, so the
number of publishable tiles is the minimum of the four counters.  The sum of the counters divided by four
is not: three warps that are two tiles ahead make it count a tile the fourth has not finished.
"""
import itertools
import random


def publishable_min(counts):
    return min(counts)


def publishable_sum(counts):
    return sum(counts) // len(counts)


def test_three_warps_ahead_do_not_publish_the_laggards_tile():
    counts = (2, 2, 2, 0)                     # warp 3 is still storing tile 0
    assert publishable_min(counts) == 0
    assert publishable_sum(counts) == 1       # the summed form would announce tile 0 too early


def test_min_rule_never_runs_ahead_of_any_warp_in_random_interleavings():
    rng = random.Random(7)
    early_by_sum = 0
    for _ in range(200):
        counts = [0, 0, 0, 0]
        tiles = 12
        published = 0
        while min(counts) < tiles:
            # a warp may advance if it is fewer than 2 tiles ahead of the slowest (two accumulator buffers)
            movable = [w for w in range(4) if counts[w] < tiles and counts[w] - min(counts) < 2]
            w = rng.choice(movable)
            counts[w] += 1
            new = publishable_min(counts)
            assert new >= published           # monotonic
            published = new
            assert all(published <= c for c in counts)
            if publishable_sum(counts) > min(counts):
                early_by_sum += 1
        assert published == tiles
    assert early_by_sum > 0                   # the interleavings do reach states the summed form gets wrong


def test_every_reachable_state_with_lead_two():
    for counts in itertools.product(range(4), repeat=4):
        if max(counts) - min(counts) > 2:
            continue
        assert publishable_min(counts) <= min(counts)
