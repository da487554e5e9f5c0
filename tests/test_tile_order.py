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


def _ctx(reqs):
    """A step's host-side description: (cached, new tokens) a request."""
    from types import SimpleNamespace
    q_start = [0]
    for _, n in reqs:
        q_start.append(q_start[-1] + n)
    return SimpleNamespace(B=len(reqs), h_q_start=q_start, h_start_pos=[c for c, _ in reqs],
                           h_slots=list(range(10, 10 + len(reqs))), scratch={})


def test_which_single_tokens_of_a_mixed_step_leave_the_portion_kernel():
    from tensorline_b200.ops_attention import _single_token_requests
    # long single contexts beside a short portion: all single tokens go, with their rows, positions and slots
    ctx = _ctx([(4000, 1), (0, 300), (50, 1), (2000, 1)])
    found = _single_token_requests(ctx, "cpu", 7)
    assert found["set"] == frozenset({0, 2, 3}) and found["span"] == 4001
    assert found["rows"].tolist() == [0, 302, 301]                              # the longest context first
    assert found["start_pos"].tolist() == [4000, 2000, 50] and found["slots"].tolist() == [10, 13, 12]
    assert _single_token_requests(ctx, "cpu", 7) is found                       # once a step
    # the portion reads about as many keys as the longest single token: one kernel for all
    assert _single_token_requests(_ctx([(4000, 1), (2048, 2041)]), "cpu", 7) is None
    # short contexts, only single tokens, no single tokens
    assert _single_token_requests(_ctx([(300, 1), (0, 100)]), "cpu", 7) is None
    assert _single_token_requests(_ctx([(4000, 1), (3000, 1)]), "cpu", 7) is None
    assert _single_token_requests(_ctx([(4000, 2), (0, 100)]), "cpu", 7) is None
    # many single tokens beside a portion that reads as many keys: their (request, KV head) pairs fill the GPU 1.6 times over
    many = [(1500, 1)] * 30 + [(1500, 482)]
    assert _single_token_requests(_ctx(many), "cpu", 5, nkv=8, sms=148)["set"] == frozenset(range(30))
    assert _single_token_requests(_ctx(many), "cpu", 7, nkv=4, sms=148) is None
    assert _single_token_requests(_ctx([(1500, 1)] * 16 + [(1500, 496)]), "cpu", 5, nkv=8, sms=148) is None


def test_skipped_requests_get_no_tile():
    order = tile_order([0, 1, 301, 302], [4000, 0, 900], 7, 128, "cpu", skip=frozenset({0, 2})).tolist()
    assert sorted(v >> 16 for v in order) == [1] * (-(-300 * 7 // 128))
    assert [v & 0xFFFF for v in order] == sorted((v & 0xFFFF for v in order), reverse=True)
    # one request left and others skipped: still an explicit order (the kernel's own would include them)
    assert tile_order([0, 1, 101], [4000, 0], 1, 64, "cpu", skip=frozenset({0})).tolist() == [(1 << 16) | 1, 1 << 16]


def test_key_ranges_of_a_decode_step_never_exceed_the_block_table_copy():
    """A decode block copies its range's block-table entries to shared memory, DECODE_MAX_TABLE_ENTRIES at most.
    Whatever page size, context and batch the engine's options allow, the planned ranges stay within that and
    cover the whole span (small pages at long contexts used to plan one range of 4,096 pages and fail at launch)."""
    from tensorline_b200.ops_attention import DECODE_MAX_TABLE_ENTRIES, KEY_TILE, plan_splits
    for page in (1, 2, 4, 8, 16, 32, 64):
        for span in (1, 63, 64, 65, 4096, 16384, 32768, 65536, 131072, 1 << 20):
            for batch in (1, 2, 8, 32, 64, 256):
                for nkv, group, d in ((4, 7, 128), (8, 5, 128), (1, 3, 32), (2, 20, 64)):
                    chunk, splits = plan_splits(batch, nkv, group, span, d, page_size=page, sms=148)
                    assert chunk % KEY_TILE == 0 and chunk > 0 and splits >= 1
                    assert chunk // page <= DECODE_MAX_TABLE_ENTRIES, (page, span, batch, chunk)
                    assert chunk * splits >= span, (page, span, batch, chunk, splits)
                    assert chunk * (splits - 1) < -(-span // KEY_TILE) * KEY_TILE          # no empty range
    # the cases that used to fail: the GPU is full, so one range took the whole span
    assert plan_splits(64, 4, 7, 32768, 128, page_size=8, sms=148) == (8192, 4)
    assert plan_splits(64, 4, 7, 65536, 128, page_size=16, sms=148) == (16384, 4)
