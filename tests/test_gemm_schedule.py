"""The CTA-pair product's schedule, checked on the host through the kernel library's own code.

`ferrum_gemm_pair_schedule` runs the same `PairSchedule` that the kernel's three roles walk
(producer, MMA issuer, epilogue).  For every pair it lists the segments (tile, k-blocks); here
they are put together again: every (tile, k-block) unit is computed exactly once, a pair leaves
at most one partial in each of its two workspace slots, the contributors of a shared tile are
exactly the consecutive pairs the kernel's owner formulas name, the pair that holds a shared
tile's first k-blocks meets it in its last segment (the finisher's stages lie idle then), and
the tile numbering reaches every (weight tile, token tile) once.  No GPU is needed: the
library is compiled here and only its host function is called.
"""
import ctypes
import random

import pytest


@pytest.fixture(scope="module")
def schedule():
    from ferrum_b200.ops import lib as ops
    fn = ops.lib().ferrum_gemm_pair_schedule
    fn.restype = ctypes.c_int
    out = (ctypes.c_longlong * 8)()

    def segments(M, rows, K, pairs, cluster):
        segs = []
        s = 0
        while fn(ctypes.c_int(M), ctypes.c_longlong(rows), ctypes.c_int(K), ctypes.c_int(pairs), ctypes.c_int(cluster),
                 ctypes.c_int(s), out):
            segs.append(tuple(out))
            s += 1
            assert s < 100000
        return segs
    return segments


def check(schedule, M, rows, K, pairs):
    nkb = (K + 63) // 64
    tiles_n, tiles_t = (rows + 255) // 256, (M + 255) // 256
    done = {}
    coords = {}
    sharers = {}
    n_shared_tiles = 0
    for c in range(pairs):
        slots = set()
        segs = schedule(M, rows, K, pairs, c)
        for i, (tile, kb0, kb1, n_idx, t_idx, first, last, slot) in enumerate(segs):
            assert 0 <= kb0 < kb1 <= nkb
            assert 0 <= n_idx < tiles_n and 0 <= t_idx < tiles_t
            assert coords.setdefault(tile, (n_idx, t_idx)) == (n_idx, t_idx)
            for kb in range(kb0, kb1):
                assert (tile, kb) not in done, f"unit {(tile, kb)} computed twice (pairs {done.get((tile, kb))} and {c})"
                done[(tile, kb)] = c
            if first >= 0:                                   # a tile that pairs share
                assert first <= c <= last and last > first
                assert slot in (0, 1) and slot not in slots, "two partials in one workspace slot"
                slots.add(slot)
                sharers.setdefault(tile, (first, last, []))[2].append(c)
                assert sharers[tile][:2] == (first, last)
                if c == first:
                    assert i == len(segs) - 1, "the finisher meets its tile before its last segment"
            else:
                assert (kb0, kb1) == (0, nkb)
    assert len(done) == tiles_n * tiles_t * nkb, "units left out"
    assert len(set(coords.values())) == tiles_n * tiles_t == len(coords), "tile numbering is not one-to-one"
    for tile, (first, last, cs) in sharers.items():
        assert cs == list(range(first, last + 1)), (tile, first, last, cs)
        n_shared_tiles += 1
    return n_shared_tiles


def test_prefill_shapes(schedule):
    """The products of a Llama-3.1-8B layer at 2048 tokens on 74 pairs: whole tiles only
    (the left-over tiles are too short to be worth cutting)."""
    for rows, K in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
        assert check(schedule, 2048, rows, K, 74) == 0


def test_long_tiles_are_cut(schedule):
    """Few tiles of many k-blocks are shared among the pairs; one wave too many joins the cut."""
    assert check(schedule, 512, 4096, 14336, 74) > 0          # 32 tiles of 224 k-blocks on 74 pairs
    assert check(schedule, 300, 256, 8192, 6) > 0
    assert check(schedule, 515, 640, 8192, 4) > 0             # 9 tiles on 4 pairs: the last whole wave is cut too
    assert check(schedule, 257, 256, 64 * 500, 74) > 0        # two tiles, dozens of sharers each


def test_random_shapes(schedule):
    rng = random.Random(7)
    for _ in range(300):
        M = rng.randint(129, 3000)
        rows = rng.randint(1, 40) * rng.choice((64, 200, 256))
        K = rng.choice((64, 320, 4096, 8192, 14336, 20000))
        check(schedule, M, rows, K, rng.randint(1, 74))
