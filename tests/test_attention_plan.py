"""How a step's rows are shared out among the attention kernels (host arithmetic only)."""
import random

from fusezap_core_b200.kernels.table import (KEY_TILE, LONG_PORTION, MAX_CUT_TILES, MAX_PIECES, PIECE_MIN_TILES, TILE_ROWS,
                                             attention_tiles)


def key_tiles_of(pos0, r, n):
    return (pos0 + min(r + TILE_ROWS, n) - 1) // KEY_TILE + 1


def check(portions, n_rows, cut=True, heads=32, items=16):
    entries, cuts, short = attention_tiles(portions, n_rows, cut, heads, items, 148)
    assert len(cuts) <= MAX_CUT_TILES
    by_row = {s: (n, p0) for s, n, p0 in portions}
    assert short == n_rows - sum(n for _, n, _ in portions if n >= LONG_PORTION)
    # every query tile of every long portion is covered exactly once: whole, or by pieces that tile its keys in order
    want = {(s, r) for s, n, _ in portions if n >= LONG_PORTION for r in range(0, n, TILE_ROWS)}
    n_pieces = sum(c for _, c in cuts)
    assert n_pieces <= MAX_PIECES and all(e[2] >= 0 for e in entries[:n_pieces]) and all(e[2] < 0 for e in entries[n_pieces:])
    seen = set()
    at = 0
    for first, count in cuts:
        assert first == at and count >= 2
        s, r, _ = entries[first]
        n, p0 = by_row[s]
        lo = 0
        for s2, r2, rng in entries[first: first + count]:
            assert (s2, r2) == (s, r) and rng & 0xffff == lo and (rng >> 16) >= 1
            lo += rng >> 16
        assert lo == key_tiles_of(p0, r, n), "the pieces cover the tile's key tiles once"
        assert min(e[2] >> 16 for e in entries[first: first + count - 1]) >= PIECE_MIN_TILES
        seen.add((s, r))
        at += count
    for s, r, rng in entries[n_pieces:]:
        assert (s, r) not in seen
        seen.add((s, r))
    assert seen == want
    return entries, cuts


def test_a_whole_prompt_is_not_cut():
    entries, cuts = check([(0, 2048, 0)], 2048)
    assert not cuts and len(entries) == 16 and entries[0][:2] == (0, 1920), "the tile with the most keys stands first"


def test_a_small_portion_of_a_long_prompt_is_cut_along_the_keys():
    entries, cuts = check([(0, 256, 32512), (1, 1, 77)], 257)
    assert len(cuts) == 2 and sum(c for _, c in cuts) == 18, "two rounds of pairs of heads for 148 SMs: 18 x 16 = 288 items"
    entries, cuts = check([(0, 256, 32512)], 256, heads=14, items=14)
    assert len(cuts) == 2 and sum(c for _, c in cuts) in (20, 21, 22)
    entries, cuts = check([(0, 256, 32512), (1, 1, 77)], 257, cut=False)
    assert not cuts and len(entries) == 2


def test_short_contexts_and_many_tiles_stay_whole():
    assert not check([(0, 256, 1000)], 256)[1]                      # 10 key tiles: too few for two pieces of eight
    assert not check([(0, 512, 5000)], 512)[1], "4 tiles x 32 heads keep most SMs busy, and the keys are few"
    assert check([(0, 512, 50000)], 512)[1], "with many keys behind them the cuts pay all the same"
    assert check([(0, 512, 5000)], 512, heads=8, items=4)[1], "4 tiles x 8 heads leave most SMs without work"
    assert not check([(0, 1280, 50000)], 1280)[1], "10 tiles x 32 heads are more than two items per SM"


def test_random_steps():
    rng = random.Random(0)
    for _ in range(300):
        portions, rows = [], 0
        for s in range(rng.randint(1, 6)):
            n = rng.choice((1, 3, 8, 40, 128, 129, 300, 700))
            portions.append((s, n, rng.choice((0, 5, 127, 1000, 5000, 40000, 300000))))
            rows += n
        heads = rng.choice((2, 8, 14, 32, 64))
        check(portions, rows + rng.randint(0, 5), True, heads, rng.choice((heads, max(1, heads // 2))))
