"""Throughput measurements of the engine at published Qwen2.5 layer sizes, random weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--model 7b|14b|32b]
                    [--workload decode|mix] [--layers L] [--profile]
    tensorline bench ...            (the same, from the installed command)

Prints ONE JSON line.  Default (`--model 7b --workload decode`): `value` is decoded tokens a second at batch 8,
timed on the device with CUDA events over exactly K decode steps (each one replay of the engine's decode
graph: its own kernels, the library matrix products, the in-graph argmax) after W warm-up steps; every request
holds a context just under the model's benchmark context, so each step streams every weight once and the cache
of the live requests, far more than the L2 holds.  `e2e` is the same metric through the Python entry point
(`Engine.step`): host token ids in, sampled token ids back on the host, every step.  `prefill` times one
2,048-token prompt as a single step (host packing and its copy included).  `roofline` divides the bytes a decode
step has to read (every weight once plus the live cache) by its time and by the measured copy bandwidth.
`points` holds decode at batch 1 and 64.

`--workload mix`: the continuous-batching mix (64 requests, prompt lengths uniform in [128, 2048], output lengths
uniform in [64, 512], one arrival per engine step, prompts cut into portions of 512 tokens) through
`Engine.add_request` / `Engine.step`; `value` is generated tokens a second of wall-clock time, `step_kinds`
the mean time of a step by what it held, `preemptions` how often the scheduler had to recompute a request.

`--profile`: after the measurement, one eager decode step and one prompt step (with `--workload mix`: one mixed step
of 48 single tokens beside a 464-token portion) with a CUDA event after every
kernel launch of this package and every library product; prints milliseconds per kernel class to stderr and
adds them to the line as `profile`.

Synthetic data: random weights N(0, 0.02), uniform random token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

def _sizes(layers, hidden, heads, kv_heads, inter, eps):
    return dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=128, intermediate_size=inter, vocab_size=152064, rope_theta=1e6,
                rms_norm_eps=eps, tie_word_embeddings=False, use_sliding_window=False, max_position_embeddings=32768,
                hidden_act="silu", eos_token_id=151645)


# Layer sizes of the published Qwen2.5 checkpoints, the context each is measured at (prompt + decoded tokens)
# and the workload it is measured with by default.
MODELS = {
    "7b": dict(name="Qwen2.5-7B", sizes=_sizes(28, 3584, 28, 4, 18944, 1e-6), context=4096, workload="decode"),
    "14b": dict(name="Qwen2.5-14B", sizes=_sizes(48, 5120, 40, 8, 13824, 1e-5), context=4096, workload="mix"),
    "32b": dict(name="Qwen2.5-32B", sizes=_sizes(64, 5120, 40, 8, 27648, 1e-5), context=3072, workload="decode"),
}
QWEN25_7B = MODELS["7b"]["sizes"]
CONTEXT = 4096
PROMPT = 2048
PAGE = 16
PREFILL_TOKENS = 2048
MIX = dict(requests=64, prompt=(128, 2048), output=(64, 512), chunk=512)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    """The roofline denominators: MEASURED_PEAKS.json beside the package or in the working directory, else the
    stated fallback."""
    out, src = dict(FALLBACK_PEAKS), "fallback"
    path = next((f for f in (os.path.join(ROOT, "MEASURED_PEAKS.json"), "MEASURED_PEAKS.json") if os.path.isfile(f)), "")
    if path:
        try:
            raw = json.load(open(path))
            for k in out:
                if isinstance(raw.get(k), (int, float)) and raw[k] > 0:
                    out[k] = float(raw[k])
            src = "measured"
        except Exception:
            pass
    return out, src


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def random_weights(cfg, device, seed=0):
    """name -> bfloat16 tensor on the device: N(0, 0.02), norm weights 1."""
    import torch
    from tensorline_b200.models import expected_tensors
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = {}
    for name, spec in expected_tensors(cfg).items():
        if spec.optional:
            continue
        if spec.init == "ones":
            out[name] = torch.ones(spec.shape, dtype=torch.bfloat16, device=device)
        else:
            t = torch.empty(spec.shape, dtype=torch.bfloat16, device=device)
            t.normal_(0.0, 0.02, generator=g)
            out[name] = t
    return out


def weight_bytes_read_per_step(cfg, layers):
    """Bytes of weights one decode step reads: every matrix of every layer once, the output head, the
    norms; embedding rows are a few KB and left out."""
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    per_layer = (nq + 2 * nkv) * d * (H + 1) + nq * d * H + 3 * H * I + 2 * H
    return 2 * (layers * per_layer + cfg.vocab_size * H + H)


def prefill_flops(cfg, layers, T):
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    linear = layers * ((nq + 2 * nkv) * d * H + nq * d * H + 3 * H * I)
    attn = layers * 4 * nq * d * (T * (T + 1) // 2)
    return 2 * T * linear + attn + 2 * cfg.vocab_size * H


def fill_context(eng, rids_tokens, chunk=2048):
    """Bring requests to their context through the runner: prompt portions of up to `chunk` tokens."""
    from tensorline_b200.engine.runner import StepEntry
    runner, cache = eng.runner, eng.cache
    for rid, toks in rids_tokens:
        assert cache.admit(rid) is not None
        runner.start_request(rid, 0)
        for s in range(0, len(toks), chunk):
            part = toks[s:s + chunk]
            assert cache.grow(rid, s, s + len(part)), "cache pool too small for the benchmark"
            runner.step([StepEntry(rid, part, [])])


def timed_decode(eng, batch, ctx0, steps, warmup, vocab, sampler=None):
    """Device-timed decode: `batch` requests at context ctx0, W + K graph-replayed steps.
    Returns (ms per step, launches of our kernels per step)."""
    import torch
    from tensorline_b200 import ops
    from tensorline_b200.engine.runner import StepEntry
    runner, cache = eng.runner, eng.cache
    g = torch.Generator().manual_seed(batch)
    reqs = [(f"bench{batch}_{i}", torch.randint(0, vocab, (ctx0,), generator=g).tolist()) for i in range(batch)]
    fill_context(eng, reqs)
    nxt = torch.randint(0, vocab, (warmup + steps, batch), generator=g).tolist()
    pos = ctx0

    def one(k):
        nonlocal pos
        entries = []
        for i, (rid, _) in enumerate(reqs):
            assert cache.grow(rid, pos, pos + 1)
            entries.append(StepEntry(rid, [nxt[k][i]], [0]))
        runner.step_graph(entries)
        pos += 1

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
        time.sleep(0.25)
    l0 = ops.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for k in range(warmup, warmup + steps):
        one(k)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = (ops.launch_count() - l0) // steps
    clocks = sampler.stop() if sampler else None
    for rid, _ in reqs:
        cache.release(rid)
        runner.end_request(rid)
    return ms, launches, clocks


def e2e_decode(eng, batch, ctx0, steps, warmup, vocab):
    """The same through `Engine.step()`: token ids from the host, sampled ids back to the host."""
    import torch
    from tensorline_b200 import SamplingParams
    g = torch.Generator().manual_seed(1000 + batch)
    prompts = [torch.randint(0, vocab, (ctx0,), generator=g).tolist() for _ in range(batch)]
    reqs = [eng.add_request(p, SamplingParams(max_tokens=1 << 20, ignore_eos=True)) for p in prompts]
    while any(r.num_computed < r.prompt_len for r in reqs):         # chunked prefill through the scheduler
        eng.step()
    for _ in range(warmup):
        eng.step()
    eng.flush()                                                     # nothing in flight when the clock starts
    torch.cuda.synchronize()
    replays0 = eng.runner.graph_replays
    before = sum(r.num_generated for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()                                                  # with overlap on, launches step t+1, then reads step t
    eng.flush()                                                     # the last step's tokens are on the host
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    produced = sum(r.num_generated for r in reqs) - before
    assert produced == batch * steps and eng.runner.graph_replays - replays0 == steps
    nb = eng.runner._bucket(batch)
    h2d = (7 * nb + 1) * 4                                          # the step's packed inputs
    d2h = nb * 4                                                    # the sampled tokens
    for r in reqs:
        eng.abort(r)
    return produced / dt, h2d, d2h


def timed_prefill(eng, tokens, vocab, iters=24, warm=4):
    """Median time of one `tokens`-token prompt step.  Under the power limit the clock of a run of such steps swings
    with a period of about ten steps (single steps of the 7B sizes read 21 to 27 ms, the first ones after a pause the
    fastest), so the median is taken over two dozen."""
    import torch
    from tensorline_b200.engine.runner import StepEntry
    runner, cache = eng.runner, eng.cache
    g = torch.Generator().manual_seed(77)
    times = []
    for it in range(warm + iters):
        toks = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        rid = f"prefill{it}"
        cache.admit(rid)
        runner.start_request(rid, 0)
        cache.grow(rid, 0, tokens)
        entry = [StepEntry(rid, toks, [tokens - 1])]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        logits = runner.step(entry)                                  # host packing and its copy are inside the timing
        end.record()
        torch.cuda.synchronize()
        assert logits.shape == (1, vocab)
        if it >= warm:
            times.append(start.elapsed_time(end))
        cache.release(rid)
        runner.end_request(rid)
    return statistics.median(times)




def mix_workload(eng, vocab, seed=0):
    """The continuous-batching mix through the public entry point: one request arrives per engine step until all
    MIX["requests"] are in; then the engine runs until the last one is done.  Returns a dictionary of figures."""
    import torch
    from tensorline_b200 import SamplingParams
    g = torch.Generator().manual_seed(seed)
    n = MIX["requests"]
    plens = torch.randint(MIX["prompt"][0], MIX["prompt"][1] + 1, (n,), generator=g).tolist()
    olens = torch.randint(MIX["output"][0], MIX["output"][1] + 1, (n,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (p,), generator=g).tolist() for p in plens]
    reqs, kinds = [], {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = 0
    while len(reqs) < n or any(not r.done for r in reqs):
        if len(reqs) < n:                                            # arrivals staggered by step
            i = len(reqs)
            reqs.append(eng.add_request(prompts[i], SamplingParams(max_tokens=olens[i], ignore_eos=True)))
        t1 = time.perf_counter()
        eng.step()
        dt = time.perf_counter() - t1
        kind = eng.last_step_kind
        k = kinds.setdefault(kind, [0, 0.0])
        k[0] += 1; k[1] += dt
        steps += 1
    eng.flush()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    generated = sum(r.num_generated for r in reqs)
    assert all(r.error is None and r.num_generated == o for r, o in zip(reqs, olens))
    st = eng.stats()
    return {"generated": generated, "prompt_tokens": sum(plens), "wall_s": wall, "steps": steps,
            "tok_s": generated / wall, "total_tok_s": (generated + sum(plens)) / wall,
            "step_kinds": {k: {"steps": c, "mean_ms": round(1000 * t / c, 3)} for k, (c, t) in sorted(kinds.items())},
            "preemptions": st["preemptions"], "max_running": st["max_running_seen"], "overlapped_steps": st["overlapped_steps"],
            "ttft_ms_mean": round(1000 * statistics.mean(r.stats.ttft_s for r in reqs), 1)}


def profile_steps(eng, vocab, batch, ctx0):
    """Milliseconds per kernel class of one eager decode step of `batch` requests at context `ctx0` and of one
    2,048-token prompt step: a CUDA event after every launch of this package's kernels and every library product;
    the time between two events goes to the later one's name.  Eager launches with their gaps, not the graph:
    shares, not absolutes."""
    import torch
    from tensorline_b200 import ops
    from tensorline_b200.engine.runner import StepEntry
    runner, cache = eng.runner, eng.cache
    g = torch.Generator().manual_seed(5)
    out = {}
    reqs = [(f"prof{i}", torch.randint(0, vocab, (ctx0,), generator=g).tolist()) for i in range(batch)]
    fill_context(eng, reqs)
    for rid, _ in reqs:
        assert cache.grow(rid, ctx0, ctx0 + 2)
    entries = [StepEntry(rid, [1], [0]) for rid, _ in reqs]
    runner.step(entries)                                             # warm
    entries = [StepEntry(rid, [2], [0]) for rid, _ in reqs]
    ops.start_profile()
    runner.step(entries)
    out[f"decode_b{batch}_eager"] = ops.stop_profile()
    for rid, _ in reqs:
        cache.release(rid); runner.end_request(rid)
    toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
    for it in range(2):
        cache.admit("profp"); runner.start_request("profp", 0); cache.grow("profp", 0, PREFILL_TOKENS)
        if it:
            ops.start_profile()
        runner.step([StepEntry("profp", toks, [PREFILL_TOKENS - 1])])
        if it:
            out[f"prefill_{PREFILL_TOKENS}"] = ops.stop_profile()
        cache.release("profp"); runner.end_request("profp")
    for what, table in out.items():
        total = sum(ms for _, ms in table.values())
        print(f"[profile] {what}: {total:.3f} ms in {sum(c for c, _ in table.values())} launches", file=sys.stderr)
        for name, (calls, ms) in sorted(table.items(), key=lambda kv: -kv[1][1]):
            print(f"[profile]   {name:34s} {calls:5d} calls {ms:9.3f} ms {100 * ms / total:5.1f} %", file=sys.stderr)
    return {what: {name: round(ms, 4) for name, (_, ms) in table.items()} for what, table in out.items()}


def profile_mixed_step(eng, vocab, singles=48, contexts=(300, 2500), cached=1024, portion=464):
    """Milliseconds per kernel class of one mixed step as the continuous-batching mix has them: `singles` requests
    that bring one token each, at contexts drawn from `contexts`, beside a prompt portion of `portion` tokens on
    `cached` earlier ones.  The step is run eagerly five times for its time (the requests' positions are put back
    between the runs, so every run writes the same cache rows) and once more with an event after every launch."""
    import torch
    from tensorline_b200 import ops
    from tensorline_b200.engine.runner import StepEntry
    runner, cache = eng.runner, eng.cache
    g = torch.Generator().manual_seed(3)
    ctxs = torch.randint(contexts[0], contexts[1] + 1, (singles,), generator=g).tolist()
    reqs = [(f"mixs{i}", torch.randint(0, vocab, (c,), generator=g).tolist()) for i, c in enumerate(ctxs)]
    fill_context(eng, reqs, chunk=512)
    ptoks = torch.randint(0, vocab, (cached + portion,), generator=g).tolist()
    fill_context(eng, [("mixp", ptoks[:cached])], chunk=512)
    for (rid, _), c in zip(reqs, ctxs):
        assert cache.grow(rid, c, c + 1)
    assert cache.grow("mixp", cached, cached + portion)
    entries = [StepEntry(rid, [7], [0]) for rid, _ in reqs] + [StepEntry("mixp", ptoks[cached:], [portion - 1])]
    start = dict(runner.positions)

    def step():
        runner.positions.update(start)
        runner.step(entries)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    ops.start_profile()
    step()
    table = ops.stop_profile()
    # the portion's kernel and the single tokens' decode kernel run side by side on two streams, and the events lie on
    # both: only the sum of the two classes is a time
    att = [k for k in table if k.startswith("attn_")]
    if len(att) > 1:
        table["attention (" + " + ".join(sorted(att)) + ", side by side)"] = (sum(table[k][0] for k in att), sum(table[k][1] for k in att))
        for k in att:
            del table[k]
    for rid, _ in reqs + [("mixp", None)]:
        cache.release(rid); runner.end_request(rid)
    total = sum(t for _, t in table.values())
    what = f"mixed step, {singles} single tokens at {contexts[0]}..{contexts[1]} keys beside {portion} tokens on {cached}"
    print(f"[profile] {what}: {ms:.3f} ms a step; with an event after every launch {total:.3f} ms in "
          f"{sum(c for c, _ in table.values())} launches", file=sys.stderr)
    for name, (calls, t) in sorted(table.items(), key=lambda kv: -kv[1][1]):
        print(f"[profile]   {name:62s} {calls:5d} calls {t:9.3f} ms {100 * t / total:5.1f} %", file=sys.stderr)
    return {"ms_per_step": round(ms, 4), "classes": {name: round(t, 4) for name, (_, t) in table.items()}}


def run_ours(a):
    import torch
    from tensorline_b200 import Engine, Qwen2Config
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "ours", "error": "no CUDA device: this engine runs on the GPU only"}))
        return 1
    model = MODELS[a.model]
    raw = dict(model["sizes"])
    layers_full = raw["num_hidden_layers"]
    if a.layers:
        raw["num_hidden_layers"] = a.layers
    cfg = Qwen2Config.from_dict(raw)
    L = cfg.num_hidden_layers
    context = model["context"]
    workload = a.workload or model["workload"]
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    pk, pk_src = peaks()
    weights = random_weights(cfg, device)
    max_seqs = max(64, a.batch)
    mix = workload == "mix"
    eng = Engine(cfg, dtype="bfloat16", weights=weights, block_size=PAGE, max_num_seqs=max_seqs,
                 max_batched_tokens=MIX["chunk"] if mix else 2048, max_model_len=context,
                 num_blocks=max_seqs * (context // PAGE), prefix_caching=False, cuda_graphs=True)
    del weights
    V = cfg.vocab_size
    K, W = a.steps, a.warmup
    ctx0 = context - (K + W) - 1                                     # the timed steps end just under the context
    batch = a.batch
    sizes = {"layers": L, "layers_full": layers_full, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
             "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": V}
    peak_tf = pk.get("bf16_tflops_sustained") or pk["bf16_tflops"]
    if mix:
        sampler = ClockSampler(0)
        mix_workload(eng, V, seed=1) if a.warm_mix else None         # a first pass warms graphs and the allocator
        sampler.start()
        m = mix_workload(eng, V, seed=0)
        clocks = sampler.stop()
        print(f"[bench] mix: {m['tok_s']:.0f} generated tok/s, {m['total_tok_s']:.0f} tok/s with prompts, "
              f"{m['steps']} steps, {m['preemptions']} preemptions", file=sys.stderr, flush=True)
        line = {
            "metric": f"continuous-batching generated tok/s ({model['name']} bf16, {MIX['requests']} requests, prompts "
                      f"U[{MIX['prompt'][0]}, {MIX['prompt'][1]}], outputs U[{MIX['output'][0]}, {MIX['output'][1]}], "
                      f"{MIX['chunk']}-token chunks)",
            "value": round(m["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": m["steps"], "warmup": int(a.warm_mix),
            "ms_per_step": round(1000 * m["wall_s"] / m["steps"], 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": dict(sizes, model=f"{model['name']} layer sizes, random weights", global_batch=MIX["requests"],
                           seq_len=context, page_size=PAGE, chunk_tokens=MIX["chunk"], parallelism="single GPU",
                           l2="inputs larger than L2 (weights and cache are re-read from HBM every step)",
                           timing="wall clock through Engine.add_request / Engine.step, one arrival per step", peaks=pk_src),
            "clocks": clocks,
            "e2e": {"value": round(m["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                    "note": "the workload runs through the public entry point: value and e2e are the same measurement"},
            "gpu_launches": None,
            "mix": {k: m[k] for k in ("generated", "prompt_tokens", "wall_s", "total_tok_s", "step_kinds", "preemptions",
                                      "max_running", "overlapped_steps", "ttft_ms_mean")},
        }
        line["mix"]["wall_s"] = round(line["mix"]["wall_s"], 3)
        line["mix"]["total_tok_s"] = round(line["mix"]["total_tok_s"], 1)
        from tensorline_b200 import ops
        line["gpu_launches"] = ops.launch_count()
        if a.profile:
            line["profile"] = {"mixed_step": profile_mixed_step(eng, V)}
        print(json.dumps(line))
        return 0
    if a.timeline:
        # the tracing build's stamps of one captured decode step (TENSORLINE_B200_TRACE=1), as a table
        from tensorline_b200 import ops_attention, ops_gemm, timeline
        tl = timeline.Timeline({"product": ops_gemm.lib(), "attn": ops_attention.attn_lib(cfg.head_dim)}, device)
        ms, _, _ = timed_decode(eng, batch, ctx0, max(K, 8), W, V)
        tl.stop()
        print(f"decode step, batch {batch}, context {ctx0}, {L} layers: {ms:.4f} ms with the stamps")
        print(timeline.table(tl.last_step(ms)))
        return 0
    if a.only == "prefill":
        pre_ms = timed_prefill(eng, PREFILL_TOKENS, V, iters=max(1, K), warm=W)
        print(json.dumps({"impl": "ours", "only": "prefill", "layers": L, "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3)}))
        return 0
    # The two timed regions run back to back on a GPU that the power limit slows as it warms (three rounds of e2e and
    # device timing in one process: 2.929 / 2.973 ms, then 2.997 / 3.003, 3.000 / 3.009): whichever comes second reads
    # a per cent or two worse.  The end-to-end figure, the one a user sees, comes first; the host adds nothing to a step
    # (launch + read-back through the runner: 2.915 against 2.896 ms).
    if a.only != "decode":
        # Requests that finish their prompt early decode while the others are still in chunked prefill,
        # so prompts are a little shorter here: every request stays under the context limit.
        e2e, h2d, d2h = e2e_decode(eng, batch, ctx0 - 3 * batch - 8, K, W, V)
        print(f"[bench] e2e b{batch}: {e2e:.0f} tok/s", file=sys.stderr, flush=True)
    ms, launches, clocks = timed_decode(eng, batch, ctx0, K, W, V, sampler=ClockSampler(0))
    value = batch * 1000.0 / ms
    print(f"[bench] decode b{batch}: {ms:.3f} ms/step, {value:.0f} tok/s", file=sys.stderr, flush=True)
    if a.only == "decode":                                           # a short run for profilers
        print(json.dumps({"impl": "ours", "only": "decode", "batch": batch, "layers": L, "ms_per_step": round(ms, 4),
                          "value": round(value, 1), "gpu_launches": launches * K}))
        return 0
    points = {}
    for b in (1, 64):
        kb = max(10, K // 2)
        ms_b, _, _ = timed_decode(eng, b, context - (kb + W) - 1, kb, W, V)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
        print(f"[bench] decode b{b}: {ms_b:.3f} ms/step", file=sys.stderr, flush=True)
    pre_ms = timed_prefill(eng, PREFILL_TOKENS, V)
    print(f"[bench] prefill {PREFILL_TOKENS}: {pre_ms:.2f} ms", file=sys.stderr, flush=True)
    flops = prefill_flops(cfg, L, PREFILL_TOKENS)
    kv_bytes = batch * (ctx0 + W + K // 2) * eng.runner.cache_bytes_per_token()
    step_bytes = weight_bytes_read_per_step(cfg, L) + kv_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {batch} ({model['name']} bf16, context {context})", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": dict(sizes, model=f"{model['name']} layer sizes, random weights", global_batch=batch, seq_len=context,
                       context_at_timed_steps=ctx0 + W, page_size=PAGE, parallelism="single GPU",
                       prefill_tokens=PREFILL_TOKENS,
                       l2="inputs larger than L2 (weights and cache are re-read from HBM every step)",
                       decode_graph=True, peaks=pk_src),
        "clocks": clocks,
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * K,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (peak_tf * 1e12), 4),
                    "frac_of_burst": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    if a.profile:
        line["profile"] = profile_steps(eng, V, batch, min(ctx0, 2048))
    print(json.dumps(line))
    return 0


def run_reference(a):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        from reference_arm import run                                # noqa: E402
    except ImportError as e:
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/reference_arm.py is not beside the package: {e}"}))
        return 0
    return run(a, QWEN25_7B, CONTEXT, PROMPT)


def main(argv=None):
    ap = argparse.ArgumentParser("bench", description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=sorted(MODELS), default="7b", help="layer sizes of this published checkpoint")
    ap.add_argument("--workload", choices=["decode", "mix"], default=None,
                    help="decode: fixed batches at a fixed context; mix: the continuous-batching mix (default: the model's own)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="decode / prefill: a short run of that phase alone (for profilers); prints its own line")
    ap.add_argument("--batch", type=int, default=8, help="decode batch of the main measurement")
    ap.add_argument("--profile", action="store_true", help="add milliseconds per kernel class of one eager decode and one prompt step (mix: of one mixed step)")
    ap.add_argument("--timeline", action="store_true",
                    help="print the time line of one captured decode step from the kernels' own stamps (needs TENSORLINE_B200_TRACE=1)")
    ap.add_argument("--no-warm-mix", dest="warm_mix", action="store_false", help="mix: time the first pass (graph capture included)")
    a = ap.parse_args(argv)
    if a.warmup < 3:
        a.warmup = 3
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.impl == "reference":
        return run_reference(a)
    return run_ours(a)
