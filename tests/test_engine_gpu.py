"""The engine end to end: greedy generation through the entry point against the plain model, under
forced chunking, forced preemption, queueing, shared prefixes and seeded sampling."""
import pytest
import torch

from tests.plain.qwen2_plain import PlainQwen2, forward, greedy_generate
from tests.tiny import CONFIGS, PAGE_SIZE, random_tokens, write_tiny

pytestmark = pytest.mark.gpu


# A and B_FULL: prompts of 1, 5, 17, 32 tokens, 8 new tokens.  B (layers 1 and 2 see a window of 24 keys, two page
# groups) and C (head size 128, group 7): prompts long enough that the window is passed and its pages given back,
# and 40 new tokens.
PROMPT_LENGTHS = {"A": (1, 5, 17, 32), "B_FULL": (1, 5, 17, 32), "B": (3, 41, 58, 70), "C": (2, 35, 60, 47)}
NEW_TOKENS = {"A": 8, "B_FULL": 8, "B": 40, "C": 40}


@pytest.fixture(scope="module", params=["A", "B_FULL", "B", "C"])
def tiny(request, tmp_path_factory):
    name = request.param
    folder = write_tiny(name, tmp_path_factory.mktemp(name))
    plain = PlainQwen2(folder)
    V = CONFIGS[name]["vocab_size"]
    prompts = [random_tokens(V, n, seed=30 + n) for n in PROMPT_LENGTHS[name]]
    want = [greedy_generate(plain, p, NEW_TOKENS[name]) for p in prompts]
    return name, folder, prompts, want, plain


@pytest.fixture(scope="module")
def tiny_a(tmp_path_factory):
    folder = write_tiny("B_FULL", tmp_path_factory.mktemp("bf"))
    plain = PlainQwen2(folder)
    prompts = [random_tokens(384, n, seed=30 + n) for n in (1, 5, 17, 32)]
    return folder, prompts, [greedy_generate(plain, p, 8) for p in prompts]


def engine(folder, dtype="float32", **kw):
    from tensorline_b200 import Engine
    opts = dict(block_size=8, num_blocks=32, max_num_seqs=8, max_model_len=128)
    opts.update(kw)
    return Engine(str(folder), dtype=dtype, **opts)


def params(n=8, **kw):
    from tensorline_b200 import SamplingParams
    return SamplingParams(max_tokens=n, ignore_eos=True, **kw)


# A, B_FULL: prompts of 1, 5, 17, 32 tokens that grow by 8: with pages of 4 (A) they hold 2+3+6+10 pages when the
# last token is computed, with pages of 8 (B_FULL) 1+2+3+5; the "forced preemption" pool holds 10.  B and C end
# with 6+11+13+14 pages of 8 and 3+5+7+6 pages of 16 in the groups that keep all keys: pools of 30 and 16.
TIGHT_POOL = {"A": 10, "B_FULL": 10, "B": 30, "C": 16}
REGIMES = {
    "plain": lambda name: {},
    "forced chunking": lambda name: dict(max_batched_tokens=4),
    "forced preemption": lambda name: dict(num_blocks=TIGHT_POOL[name], prefix_caching=False),
    "queueing": lambda name: dict(max_num_seqs=2),
    "no graphs": lambda name: dict(cuda_graphs=False),
}


_LAST_LOGITS: dict = {}         # (plain model, sequence) -> the plain model's logits at its last position


def follows_where_decided(plain, prompt, tokens) -> int:
    """The bfloat16 rule, at every generated position: given the tokens before it (the engine's own), the engine's
    token must be one the plain model could have picked within the stated logit tolerance: its plain logit lies
    within twice the tolerance of the plain model's largest.  Where the plain model's lead over its runner-up is
    larger than that (a decided position) this means the very same token.  Returns the number of decided positions."""
    from tests.gpu_helpers import BF16_MODEL_REL
    seq, decided = list(prompt), 0
    for tok in tokens:
        key = (id(plain), tuple(seq))
        if key not in _LAST_LOGITS:
            _LAST_LOGITS[key] = forward(plain, seq)[-1]
        logits = _LAST_LOGITS[key]
        slack = 2 * BF16_MODEL_REL * float(logits.abs().max())
        top = torch.topk(logits, 2).values
        assert float(logits[tok]) >= float(top[0]) - slack, \
            f"position {len(seq)}: engine picked {tok} (plain logit {float(logits[tok]):.4f}), plain {int(logits.argmax())} ({float(top[0]):.4f})"
        decided += float(top[0] - top[1]) > slack
        seq.append(tok)
    return decided


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("regime", sorted(REGIMES))
def test_greedy_generation_equals_the_plain_model(tiny, regime, dtype):
    """tzar-beep/Tensorline's tests/test_batching.py:67-85 with tokens in place of text, in both precisions, for the
    full-attention models, the window model (two page groups, pages given back behind the window) and head size 128."""
    name, folder, prompts, want, plain = tiny
    n_new = NEW_TOKENS[name]
    opts = dict(block_size=PAGE_SIZE[name], num_blocks=64, max_model_len=160)
    opts.update(REGIMES[regime](name))
    eng = engine(folder, dtype=dtype, **opts)
    outs = eng.generate(prompts, params(n_new))
    if dtype == "float32":
        assert [o.token_ids for o in outs] == want
    else:
        decided = sum(follows_where_decided(plain, p, o.token_ids) for p, o in zip(prompts, outs))
        assert decided >= n_new // 2, "too few positions where the plain model is decided: the comparison says little"
    assert all(o.finish_reason == "length" and o.stats.completion_tokens == n_new for o in outs)
    st = eng.stats()
    assert st["free_pages"] == st["num_pages"], "pages leaked"
    assert all(eng.cache.num_free_pages(g.index) == g.pool.num_pages for g in eng.cache.groups)
    if regime == "forced preemption":
        assert st["preemptions"] > 0
    if regime == "queueing":
        assert st["max_running_seen"] == 2
    if regime == "plain":
        assert st["max_running_seen"] > 1 and st["graph_replays"] > 0
    if regime == "no graphs":
        assert st["graph_replays"] == 0



def test_bfloat16_engine_at_head_size_128_with_graphs_and_without(tmp_path):
    """Head size 128 in groups of 7, pages of 16, six requests: the decode steps take the TMA attention with the
    merge inside clusters, captured in CUDA graphs with dependent launches and overlapped scheduling.  The same
    engine without graphs must give the same tokens, and both follow the plain model where it is decided."""
    from tests.gpu_helpers import BF16_MODEL_REL
    folder = write_tiny("C", tmp_path / "c")
    plain = PlainQwen2(folder)
    V = CONFIGS["C"]["vocab_size"]
    prompts = [random_tokens(V, n, seed=70 + n) for n in (3, 150, 47, 66, 80, 34)]
    outs = {}
    for graphs in (True, False):
        eng = engine(folder, dtype="bfloat16", block_size=PAGE_SIZE["C"], num_blocks=96, max_model_len=512,
                     cuda_graphs=graphs, overlap=graphs)
        outs[graphs] = [o.token_ids for o in eng.generate(prompts, params(12))]
        st = eng.stats()
        assert st["free_pages"] == st["num_pages"]
        assert (st["graph_replays"] > 0) == graphs
    assert outs[True] == outs[False]
    assert sum(follows_where_decided(plain, p, toks) for p, toks in zip(prompts, outs[True])) >= 12


def test_request_that_does_not_fit_fails_and_others_go_on(tiny_a):
    from tensorline_b200.engine import RequestDoesNotFit
    folder, prompts, want = tiny_a
    eng = engine(folder, num_blocks=2, prefix_caching=False)
    with pytest.raises(RequestDoesNotFit):
        eng.generate([prompts[2]], params())                 # 17 tokens, 16 fit
    assert eng.generate([prompts[1]], params(3))[0].token_ids == want[1][:3]
    assert eng.stats()["free_pages"] == 2
    with pytest.raises(ValueError, match="max_model_len"):
        eng.add_request(list(range(128)))


def test_stop_token_ends_a_request_and_is_not_returned(tiny_a):
    from tensorline_b200 import SamplingParams
    folder, prompts, want = tiny_a
    eng = engine(folder)
    seq = want[3]
    k = next(i for i in range(1, 8) if seq[i] not in seq[:i])     # a token that first appears at place k
    out = eng.generate([prompts[3]], SamplingParams(max_tokens=8, stop_token_ids={seq[k]}))[0]
    assert out.token_ids == seq[:k] and out.finish_reason == "stop"


@pytest.mark.parametrize("name,dtype", [("B_FULL", "float32"), ("B_FULL", "bfloat16"), ("B", "float32"), ("B", "bfloat16")])
def test_shared_prefix_is_served_from_the_cache_and_changes_nothing(tmp_path, name, dtype):
    """tests/test_prefix_cache.py:42-74 of tzar-beep/Tensorline, on the untied group-3 model, and on the window model,
    where the window group hands over only the pages its window still reaches.  The shared prefix is 32 tokens
    (four pages), longer than the window of 24."""
    folder = write_tiny(name, tmp_path / "b")
    plain = PlainQwen2(folder)
    shared = random_tokens(384, 32, seed=1)
    prompts = [shared + random_tokens(384, n, seed=2 + n) for n in (7, 24, 48)]
    opts = dict(block_size=8, num_blocks=48, max_model_len=256)
    ref = engine(folder, dtype=dtype, prefix_caching=False, **opts).generate(prompts, params(12))
    eng = engine(folder, dtype=dtype, **opts)
    assert eng.cache.prefix_caching
    first = eng.generate([prompts[0]], params(12))
    outs = eng.generate(prompts[1:], params(12))
    if dtype == "float32":
        assert [o.token_ids for o in first + outs] == [o.token_ids for o in ref]
        assert [o.token_ids for o in ref] == [greedy_generate(plain, p, 12) for p in prompts]
    else:                                                    # a cached prefix was computed in another batch: rounding may differ
        assert sum(follows_where_decided(plain, p, o.token_ids) for p, o in zip(prompts, first + outs)) >= 6
    assert first[0].stats.cached_tokens == 0 and all(o.stats.cached_tokens == 32 for o in outs)
    again = eng.generate([prompts[1]], params(12))[0]        # found whole in the cache: the last page is computed again
    assert 0 < again.stats.cached_tokens < len(prompts[1])
    if dtype == "float32":
        assert again.token_ids == ref[1].token_ids
    st = eng.stats()
    assert st["free_pages"] == 48 and st["prefix_hit_tokens"] > 0
    assert all(eng.cache.num_free_pages(g.index) == g.pool.num_pages for g in eng.cache.groups)


def test_seeded_sampling_does_not_depend_on_batching_or_preemption(tmp_path):
    """Temperature 0.8, top-p 0.9, seeded: the same tokens alone, in a batch, and under preemption."""
    folder = write_tiny("B", tmp_path / "b")
    prompts = [random_tokens(384, n, seed=60 + n) for n in (7, 40, 64)]
    sp = [params(12, temperature=0.8, top_p=0.9, seed=1000 + i) for i in range(3)]
    opts = dict(block_size=8, max_model_len=256)
    alone = [engine(folder, num_blocks=40, **opts).generate([p], s)[0].token_ids for p, s in zip(prompts, sp)]
    together = engine(folder, num_blocks=40, **opts).generate(prompts, sp)
    assert [o.token_ids for o in together] == alone
    tight = engine(folder, num_blocks=16, **opts)
    squeezed = tight.generate(prompts, sp)
    assert [o.token_ids for o in squeezed] == alone and tight.stats()["preemptions"] > 0
    assert len({tuple(t) for t in alone}) == 3 and all(len(t) == 12 for t in alone)
    greedy = engine(folder, num_blocks=40, **opts).generate([prompts[0]], params(12))[0].token_ids
    assert greedy != alone[0]


def test_overlapped_decoding_equals_synchronous(tiny_a):
    """tzar-beep/Tensorline's tests/test_cuda_graphs.py:62-101: launching step t+1 before reading step t
    changes no token, finish reason or count, with stop tokens, limits and staggered arrivals."""
    from tensorline_b200 import SamplingParams
    folder, prompts, want = tiny_a
    stop = {want[3][5]}
    sp = [params(8), SamplingParams(max_tokens=3, ignore_eos=True), params(8), SamplingParams(max_tokens=8, stop_token_ids=stop)]
    results = {}
    for overlap in (False, True):
        eng = engine(folder, overlap=overlap)
        reqs = [eng.add_request(prompts[0], sp[0]), eng.add_request(prompts[1], sp[1])]
        for _ in range(4):                               # the other two arrive while these decode
            eng.step()
        reqs += [eng.add_request(prompts[2], sp[2]), eng.add_request(prompts[3], sp[3])]
        while any(not r.done for r in reqs):
            eng.step()
        results[overlap] = [(r.output_tokens, r.stats.finish_reason, r.stats.completion_tokens) for r in reqs]
        st = eng.stats()
        assert st["free_pages"] == st["num_pages"]
        assert (st["overlapped_steps"] > 0) == overlap
    assert results[True] == results[False]
    assert results[True][0][0] == want[0] and results[True][1][0] == want[1][:3]
    assert results[True][3][1] == "stop" and results[True][3][0] == want[3][:want[3].index(want[3][5])]


def test_overlapped_decoding_with_sampled_requests_equals_synchronous(tiny_a):
    """Sampled requests go on overlapped as well (a draw's uniform number is known a step ahead; the sampling
    kernel runs behind the decode graph): greedy and seeded temperature / top-p requests side by side give the
    same tokens with the overlap on and off, with a stop token and a length limit on the way."""
    from tensorline_b200 import SamplingParams
    folder, prompts, want = tiny_a
    sampled = dict(temperature=0.9, top_p=0.85, ignore_eos=True)
    results = {}
    for overlap in (False, True):
        eng = engine(folder, overlap=overlap)
        sp = [SamplingParams(max_tokens=10, seed=7, **sampled), params(8),
              SamplingParams(max_tokens=4, seed=8, **sampled), SamplingParams(max_tokens=9, seed=9, temperature=0.7, ignore_eos=True)]
        reqs = [eng.add_request(p, s) for p, s in zip(prompts, sp)]
        while any(not r.done for r in reqs):
            eng.step()
        results[overlap] = [(r.output_tokens, r.stats.finish_reason) for r in reqs]
        st = eng.stats()
        assert st["free_pages"] == st["num_pages"]
        assert (st["overlapped_steps"] > 0) == overlap
    assert results[True] == results[False]
    assert results[True][1][0] == want[1]                                   # the greedy one beside them is untouched
    assert [len(t) for t, _ in results[True]] == [10, 8, 4, 9]
    # a stop token drawn by a sampled request ends it there, overlapped or not
    stop = results[True][0][0][6]
    outs = {}
    for overlap in (False, True):
        eng = engine(folder, overlap=overlap)
        outs[overlap] = eng.generate([prompts[0]], SamplingParams(max_tokens=10, seed=7, temperature=0.9, top_p=0.85,
                                                                  stop_token_ids={stop}))[0]
    first = results[True][0][0].index(stop)
    assert outs[True].token_ids == outs[False].token_ids == results[True][0][0][:first]
    assert outs[True].finish_reason == outs[False].finish_reason == "stop"


def test_the_smoke_entry_point_passes():
    """`__graft_entry__.smoke()` is what a deployment check runs first: the tiny model in both precisions against the
    plain model, then one call of each Blackwell kernel family."""
    import importlib.util
    import pathlib
    path = pathlib.Path(__file__).resolve().parent.parent / "__graft_entry__.py"
    spec = importlib.util.spec_from_file_location("graft_entry_under_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.smoke()
