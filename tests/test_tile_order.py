"""The order in which prompt-portion attention takes the query tiles of several requests (host side only)."""
import random

from tensorline_b200.ops_attention import tile_order


def test_one_request_keeps_the_kernels_own_order():
    assert tile_order([0, 500], [0], 7, 128, "cpu") is None


def test_every_tile_once_and_the_longest_first():
    rng = random.Random(3)
    for _ in range(50):
        B = rng.randint(2, 6)
        group, rows_per_tile = rng.choice([1, 2, 7]), rng.choice([64, 128, 256])
        lens = [rng.randint(1, 900) for _ in range(B)]
        pos = [rng.choice([0, 0, rng.randint(1, 5000)]) for _ in range(B)]
        q_start = [0]
        for n in lens:
            q_start.append(q_start[-1] + n)
        order = tile_order(q_start, pos, group, rows_per_tile, "cpu").tolist()
        seen = [(v >> 16, v & 0xFFFF) for v in order]
        want = [(b, t) for b in range(B) for t in range(-(-lens[b] * group // rows_per_tile))]
        assert sorted(seen) == want
        keys = [pos[b] + (min(lens[b] * group, (t + 1) * rows_per_tile) - 1) // group + 1 for b, t in seen]
        assert keys == sorted(keys, reverse=True)
