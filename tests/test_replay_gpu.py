"""Trace replay against the plain implementation, in 32-bit and in bfloat16.

The same requests are replayed whole; with the last 32 tokens decoded one by one; in portions of
changing size, down to two tokens; and mixed: up to four live requests, portions of some beside
decoded tokens of others, in a pool so small that pages are given back and used again.  Every logit
of every position is compared with the plain whole-sequence model.  In 32-bit the engine's kernels
use one fixed order of additions per position, so the schedules must also agree with each other
bit for bit; a difference that appears under one way of cutting only is a fault of the cache or
of the batch.
"""
import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.gpu_helpers import BF16_MODEL_REL, BF16_MODEL_REL_OF
from tests.plain.qwen2_plain import PlainQwen2, forward
from tests.tiny import CONFIGS, PAGE_SIZE, random_tokens, write_tiny

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
LENGTHS = {"A": [1, 5, 17, 70, 33, 45, 64], "B": [7, 40, 64, 97, 35, 128, 50], "C": [3, 130, 47, 66, 80, 34]}
F32_ATOL = 3e-5                    # float32 engine against the float64 plain model, logits of order one


@pytest.fixture(scope="module", params=["A", "B", "C"])
def model(request, tmp_path_factory):
    name = request.param
    folder = write_tiny(name, tmp_path_factory.mktemp(f"tiny_{name}"))
    plain = PlainQwen2(folder)
    V = CONFIGS[name]["vocab_size"]
    reqs = {f"r{i}": random_tokens(V, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
    want = {rid: forward(plain, toks) for rid, toks in reqs.items()}
    return dict(name=name, folder=folder, reqs=reqs, want=want, page=PAGE_SIZE[name], vocab=V)


def replay(model, dtype, steps, max_tokens, graphs=False, before=None, after=None):
    """Runs trace records through the engine's own trace session; returns {(rid, position): logits}.
    `before(runner)` / `after(runner)` run around the steps (the graph tests plant and check bystanders)."""
    from tensorline_b200.replay import TraceSession, make_runner
    runner, _ = make_runner(model["folder"], dtype, max_tokens, page_size=model["page"], graphs=graphs)
    session = TraceSession(runner)
    got, pos = {}, {}
    if before:
        before(runner)
    for rec in steps:
        logits = session.run_step(rec).double().cpu()
        row = 0
        for e in rec["entries"]:
            start = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], start + w)] = logits[row]
                row += 1
            pos[e["id"]] = start + len(e["tokens"])
        assert row == logits.shape[0]
        for rid in rec["end"]:
            pos.pop(rid, None)
        runner.cache.check()
    if after:
        after(runner)
    assert all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups), "pages leaked"
    return got


def check(model, dtype, got, what):
    assert got, "nothing was compared"
    for (rid, p), row in got.items():
        ref = model["want"][rid][p]
        err = float((row - ref).abs().max())
        if dtype == "float32":
            assert err <= F32_ATOL, f"{what}: request {rid} position {p}: max abs err {err:.3e}"
        else:
            bound = BF16_MODEL_REL_OF.get(model["name"], BF16_MODEL_REL) * float(model["want"][rid].abs().max())
            assert err <= bound, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {bound:.3e}"


def steps_alone(model, cuts_of):
    """Each request alone; cuts_of(n) -> list of portion sizes."""
    steps = []
    for rid, toks in model["reqs"].items():
        s = 0
        cuts = cuts_of(len(toks))
        assert sum(cuts) == len(toks)
        for i, n in enumerate(cuts):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[s:s + n], "want": list(range(n))}],
                          "end": [rid] if i == len(cuts) - 1 else []})
            s += n
    return steps


def cuts_whole(n):
    return [n]


def cuts_last32(n):
    tail = min(32, n - 1) if n > 1 else 0
    return ([n - tail] if n - tail else []) + [1] * tail


def cuts_changing(n):
    sizes, out, i = [7, 2, 13, 2, 3, 2, 29, 4, 2, 16, 1, 5], [], 0
    while n:
        k = min(sizes[i % len(sizes)], n)
        if n - k == 1:                    # do not leave a lone token: portions go down to two
            k = n if k + 1 > 2 else k
        out.append(k)
        n -= k
        i += 1
    return out


def steps_mixed(model, seed, max_live=4):
    """Up to `max_live` live requests; portions of some beside decoded tokens of others; a request
    may be left out of a step.  Returns (steps, largest number of tokens held at any time, rounded
    up per request to whole pages)."""
    rng = random.Random(seed)
    reqs, page = model["reqs"], model["page"]
    pending, live, steps, peak = list(reqs), {}, [], 0
    while pending or live:
        while pending and len(live) < max_live and (not live or rng.random() < 0.7):
            live[pending.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            toks, done = reqs[rid], live[rid]
            decode_from = max(1, len(toks) - 8)          # the last 8 tokens come one by one
            n = min(rng.choice([2, 3, 5, 9, 16, 31]), decode_from - done) if done < decode_from else 1
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            live[rid] = done + n
            if live[rid] == len(toks):
                end.append(rid)
        if not entries:
            continue
        peak = max(peak, sum(-(-n // page) * page for n in live.values()))
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for rid in end:
            del live[rid]
    return steps, peak


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_schedules_agree_with_the_plain_model(model, dtype):
    results = {}
    for what, cuts in (("whole", cuts_whole), ("last 32 one by one", cuts_last32), ("changing portions", cuts_changing)):
        results[what] = replay(model, dtype, steps_alone(model, cuts), max_tokens=192)
        check(model, dtype, results[what], what)
        assert len(results[what]) == sum(len(t) for t in model["reqs"].values())
    for seed in (1, 2):
        steps, peak = steps_mixed(model, seed)
        assert max(len(s["entries"]) for s in steps) >= 3
        total = sum(-(-len(t) // model["page"]) * model["page"] for t in model["reqs"].values())
        assert peak < total, "the pool must be too small to hold all requests: pages have to be used again"
        results[f"mixed {seed}"] = replay(model, dtype, steps, max_tokens=peak)
        check(model, dtype, results[f"mixed {seed}"], f"mixed {seed}")
        assert len(results[f"mixed {seed}"]) == len(results["whole"])
    if dtype == "float32":                                  # one order of additions per position
        for what, got in results.items():
            for key, row in got.items():
                assert torch.equal(row, results["whole"][key]), f"{what} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(model, dtype):
    """A one-token prompt, then 150 tokens decoded one by one across many page edges."""
    V = model["vocab"]
    toks = random_tokens(V, 151, seed=7)
    want = forward(PlainQwen2(model["folder"]), toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    steps[-1]["end"] = ["x"]
    m2 = dict(model, reqs={"x": toks}, want={"x": want})
    got = replay(m2, dtype, steps, max_tokens=160)
    check(m2, dtype, got, "token by token")
    assert sorted(p for _, p in got) == list(range(151))


def steps_decode_together(model, rids, tail):
    """The requests `rids`: prompts in portions that share steps, then the last `tail` tokens of all of them one
    by one in common steps of single tokens; requests end at different steps, so the batch shrinks."""
    reqs = model["reqs"]
    steps, done = [], {r: 0 for r in rids}
    heads = {r: max(1, len(reqs[r]) - tail - i) for i, r in enumerate(rids)}      # decoding starts at different places
    while any(done[r] < heads[r] for r in rids):
        entries = []
        for r in rids:
            n = min(11, heads[r] - done[r])
            if n > 0:
                entries.append({"id": r, "tokens": reqs[r][done[r]:done[r] + n], "want": list(range(n))})
                done[r] += n
        steps.append({"step": len(steps), "entries": entries, "end": []})
    decode_steps = 0
    while any(done[r] < len(reqs[r]) for r in rids):
        entries, end = [], []
        for r in rids:
            if done[r] < len(reqs[r]):
                entries.append({"id": r, "tokens": [reqs[r][done[r]]], "want": [0]})
                done[r] += 1
                if done[r] == len(reqs[r]):
                    end.append(r)
        steps.append({"step": len(steps), "entries": entries, "end": end})
        decode_steps += 1
    return steps, decode_steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_agree_with_eager_steps_and_the_plain_model_and_touch_no_other_page(model, dtype):
    """Decode steps replayed from CUDA graphs (tzar-beep/Tensorline's tests/test_cuda_graphs.py:20-45): three live
    requests in the bucket of four (one padding row), then six in the bucket of eight, shrinking as requests end.
    Every logit against the plain model; in 32-bit bit-equal to the same steps run eagerly.  A bystander request that
    is live but in no step, and a page filled with a sentinel that no stepped request owns, must come out bit for bit
    as they went in: padding rows write to the sink page only."""
    rids = [r for r in model["reqs"] if len(model["reqs"][r]) >= 17]
    name = model["name"]
    watched = {}

    def plant(runner):
        from tensorline_b200.engine.runner import StepEntry
        from tensorline_b200.parts import KVCacheView
        cache = runner.cache
        cache.admit("bystander"); runner.start_request("bystander", 0)
        toks = random_tokens(model["vocab"], 2 * model["page"] + 1, seed=5)
        assert cache.grow("bystander", 0, len(toks))
        runner.step([StepEntry("bystander", toks, [])])
        cache.admit("sentinel"); runner.start_request("sentinel", 0)
        assert cache.grow("sentinel", 0, 1)
        for cid, view in runner.caches.items():
            if isinstance(view, KVCacheView):
                g = view.group
                for p in cache.pages("sentinel", g):
                    view.k[p].fill_(7.0); view.v[p].fill_(-7.0)
                pages = [p for p in cache.pages("bystander", g) + cache.pages("sentinel", g) if p >= 0]
                watched[cid] = (pages, view.k[pages].clone(), view.v[pages].clone())

    def verify(runner):
        assert watched
        for cid, (pages, k, v) in watched.items():
            view = runner.caches[cid]
            assert torch.equal(view.k[pages], k) and torch.equal(view.v[pages], v), f"cache {cid}: a bystander page changed"
        for rid in ("bystander", "sentinel"):
            runner.cache.release(rid); runner.end_request(rid)
        assert runner.graph_replays >= 1

    spare = (2 * model["page"] + 1 + model["page"] - 1) // model["page"] * model["page"] + model["page"]
    for group, tail in ((rids[:3], 32), (rids[:6] if len(rids) >= 6 else rids, 10)):
        if len(group) < 3:
            continue
        steps, decode_steps = steps_decode_together(dict(model), group, tail)
        assert decode_steps >= tail
        room = sum(-(-len(model["reqs"][r]) // model["page"]) * model["page"] for r in group) + spare
        m2 = dict(model, reqs={r: model["reqs"][r] for r in group})
        eager = replay(m2, dtype, steps, room)
        counted = {}

        def verify_and_count(runner):
            verify(runner)
            counted["replays"] = runner.graph_replays
            counted["buckets"] = sorted(runner._graphs)
        graphed = replay(m2, dtype, steps, room, graphs=True, before=plant, after=verify_and_count)
        assert counted["replays"] >= decode_steps
        assert len(group) in (3, 5, 6, 7) and max(counted["buckets"]) > len(group)      # padding rows were there
        check(m2, dtype, graphed, f"graphs, {len(group)} requests, {name}")
        assert graphed.keys() == eager.keys()
        if dtype == "float32":
            for key in graphed:
                assert torch.equal(graphed[key], eager[key]), f"graph replay differs from the eager step at {key}"
        else:
            scale = max(float(w.abs().max()) for w in model["want"].values())
            worst = max(float((graphed[k] - eager[k]).abs().max()) for k in graphed)
            assert worst <= BF16_MODEL_REL_OF.get(name, BF16_MODEL_REL) * scale


def test_pool_that_is_too_small_is_reported(model):
    toks = model["reqs"]["r3"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": []}]
    with pytest.raises(RuntimeError, match="exhausted"):
        replay(model, "float32", steps, max_tokens=model["page"])


def test_trace_run_program(model, tmp_path):
    """The program itself: JSON lines in, `done <step>` lines and <step>.f32 files out."""
    if model["name"] != "B":
        pytest.skip("one configuration is enough for the command-line protocol")
    reqs = model["reqs"]
    a, b = reqs["r1"], reqs["r2"]
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:9], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[30:], "want": [len(a) - 31]},
                                {"id": "b", "tokens": b[9:11], "want": [1]}], "end": ["a"]},
        {"step": 5, "entries": [{"id": "b", "tokens": b[11:], "want": [len(b) - 12]}], "end": ["b"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model["folder"]),
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128", "--page-size", "8"],
                          input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 5"]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "2.f32", "5.f32"]
    V = model["vocab"]
    s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    s2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    s5 = np.fromfile(out / "5.f32", dtype="<f4").reshape(-1, V)
    assert s0.shape[0] == 2 and s2.shape[0] == 2 and s5.shape[0] == 1
    wa, wb = model["want"]["r1"], model["want"]["r2"]
    for got, ref in ((s0[0], wa[0]), (s0[1], wa[29]), (s2[0], wa[-1]), (s2[1], wb[10]), (s5[0], wb[-1])):
        assert float((torch.from_numpy(got.astype(np.float64)) - ref).abs().max()) <= F32_ATOL
