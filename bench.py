#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes, random weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Prints ONE JSON line.  `value` is decoded tokens a second at batch 8, timed on the device with CUDA
events over exactly K decode steps (each one replay of the engine's decode graph: its own kernels,
the library matrix products, the in-graph argmax) after W warm-up steps; every request holds a
context just under 4,096 tokens, so each step streams every weight once and the cache of the live
requests, far more than the L2 holds.  `e2e` is the same metric through the Python entry point
(`Engine.step`): host token ids in, sampled token ids back on the host, every step.  `prefill` times
one 2,048-token prompt as a single step.  `roofline` divides the bytes a decode step has to read
(every weight once plus the live cache) by its time and by the measured copy bandwidth.  `points`
holds decode at batch 1 and 64.  Synthetic data: random weights N(0, 0.02), uniform random token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-7B layer sizes (BASELINE.json configs[2])
QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
                 num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6,
                 rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
                 max_position_embeddings=32768, hidden_act="silu", eos_token_id=151645)
CONTEXT = 4096
PROMPT = 2048
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out, src = dict(FALLBACK_PEAKS), "fallback"
    if os.path.isfile(path):
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


def timed_prefill(eng, tokens, vocab, iters=5, warm=3):
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
        ctx = runner.build_context(entry)                            # host work and copies outside the timing
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        with torch.inference_mode():
            logits = runner.model.forward(ctx, runner.caches)
        end.record()
        torch.cuda.synchronize()
        assert logits.shape == (1, vocab)
        if it >= warm:
            times.append(start.elapsed_time(end))
        cache.release(rid)
        runner.end_request(rid)
    return statistics.median(times)


def run_ours(a):
    import torch
    from tensorline_b200 import Engine, Qwen2Config
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "ours", "error": "no CUDA device: this engine runs on the GPU only"}))
        return 1
    raw = dict(QWEN25_7B)
    layers_full = raw["num_hidden_layers"]
    if a.layers:
        raw["num_hidden_layers"] = a.layers
    cfg = Qwen2Config.from_dict(raw)
    L = cfg.num_hidden_layers
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    pk, pk_src = peaks()
    weights = random_weights(cfg, device)
    max_seqs = max(64, a.batch)
    eng = Engine(cfg, dtype="bfloat16", weights=weights, block_size=PAGE, max_num_seqs=max_seqs,
                 max_batched_tokens=2048, max_model_len=CONTEXT, num_blocks=max_seqs * (CONTEXT // PAGE),
                 prefix_caching=False, cuda_graphs=True)
    del weights
    V = cfg.vocab_size
    K, W = a.steps, a.warmup
    ctx0 = CONTEXT - (K + W) - 1                                     # the timed steps end just under 4,096
    batch = a.batch
    if a.only == "prefill":
        pre_ms = timed_prefill(eng, PREFILL_TOKENS, V, iters=max(1, K), warm=W)
        print(json.dumps({"impl": "ours", "only": "prefill", "layers": L, "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3)}))
        return 0
    ms, launches, clocks = timed_decode(eng, batch, ctx0, K, W, V, sampler=ClockSampler(0))
    value = batch * 1000.0 / ms
    print(f"[bench] decode b{batch}: {ms:.3f} ms/step, {value:.0f} tok/s", file=sys.stderr, flush=True)
    # Requests that finish their prompt early decode while the others are still in chunked prefill,
    # so prompts are a little shorter here: every request stays under the 4,096-token limit.
    if a.only == "decode":                                           # a short run for profilers
        print(json.dumps({"impl": "ours", "only": "decode", "batch": batch, "layers": L, "ms_per_step": round(ms, 4),
                          "value": round(value, 1), "gpu_launches": launches * K}))
        return 0
    e2e, h2d, d2h = e2e_decode(eng, batch, ctx0 - 3 * batch - 8, K, W, V)
    print(f"[bench] e2e b{batch}: {e2e:.0f} tok/s", file=sys.stderr, flush=True)
    points = {}
    for b in (1, 64):
        kb = max(10, K // 2)
        ms_b, _, _ = timed_decode(eng, b, CONTEXT - (kb + W) - 1, kb, W, V)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
        print(f"[bench] decode b{b}: {ms_b:.3f} ms/step", file=sys.stderr, flush=True)
    pre_ms = timed_prefill(eng, PREFILL_TOKENS, V)
    print(f"[bench] prefill {PREFILL_TOKENS}: {pre_ms:.2f} ms", file=sys.stderr, flush=True)
    flops = prefill_flops(cfg, L, PREFILL_TOKENS)
    peak_tf = pk.get("bf16_tflops_sustained") or pk["bf16_tflops"]
    kv_bytes = batch * (ctx0 + W + K // 2) * eng.runner.cache_bytes_per_token()
    step_bytes = weight_bytes_read_per_step(cfg, L) + kv_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {batch} (Qwen2.5-7B bf16, context 4096)", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen2.5-7B layer sizes, random weights", "layers": L, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": V,
                   "global_batch": batch, "seq_len": CONTEXT, "context_at_timed_steps": ctx0 + W,
                   "page_size": PAGE, "parallelism": "single GPU", "prefill_tokens": PREFILL_TOKENS,
                   "l2": "inputs larger than L2 (weights and cache are re-read from HBM every step)",
                   "decode_graph": True, "peaks": pk_src},
        "clocks": clocks,
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * K,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (peak_tf * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def run_reference(a):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    from reference_arm import run                                    # noqa: E402
    return run(a, QWEN25_7B, CONTEXT, PROMPT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="decode / prefill: a short run of that phase alone (for profilers); prints its own line")
    ap.add_argument("--batch", type=int, default=8, help="decode batch of the main measurement")
    a = ap.parse_args()
    if a.warmup < 3:
        a.warmup = 3
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.impl == "reference":
        return run_reference(a)
    return run_ours(a)


if __name__ == "__main__":
    sys.exit(main())
