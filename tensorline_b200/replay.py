"""Trace replay: feed given token ids through a model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--graphs]

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through the engine's own step function (`ModelRunner.step`),
model, cache manager and kernels: the ones generation uses.  Nothing is sampled.  For a step
in which logits are wanted, `OUT/<step>.f32` holds them as little-endian float32
[wanted, vocab], in the order of the entries and of `want`.  After every step a line
`done <step>` is printed and flushed.  `end` names the requests that are finished after the step;
their pages and slots are given back and used again.  The cache pool holds `--max-tokens` tokens
(each live request's count rounded up to whole pages), and not one page more.  With `--graphs`, a
step whose entries are all single tokens of running requests with `want` [0] (a decode step) is
replayed from the CUDA graph of its batch-size bucket, as generation does; every other step runs
as it is.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def make_runner(model_dir, dtype: str, max_tokens: int, *, page_size: int = 16, max_live: int = 8, graphs: bool = False):
    import torch

    from .cache import CacheManager
    from .engine.runner import ModelRunner
    from .models import load_model
    from .parts import Runtime

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs on the GPU only")
    device = torch.device("cuda", torch.cuda.current_device())
    act = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    rt = Runtime(device, act, page_size)
    model, cfg = load_model(model_dir, rt)
    num_pages = max(1, -(-max_tokens // page_size))
    cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=num_pages, max_num_seqs=max_live,
                         max_model_len=num_pages * page_size, prefix_caching=False)
    runner = ModelRunner(model, cache)
    runner.use_graphs = bool(graphs)
    return runner, cfg


class TraceSession:
    """Feeds trace records to a runner, one step at a time; what `main` does for every line."""

    def __init__(self, runner):
        self.runner = runner
        self.cache = runner.cache

    def run_step(self, rec: dict):
        """Run one record; returns the logits [wanted, vocab] on the device (may be empty)."""
        from .engine.runner import StepEntry

        cache, runner = self.cache, self.runner
        entries = []
        for e in rec.get("entries", []):
            rid, toks = e["id"], e["tokens"]
            if not cache.holds(rid):
                if cache.admit(rid) is None:
                    raise RuntimeError(f"step {rec['step']}: more than {cache.max_num_seqs} live requests")
                runner.start_request(rid, 0)
            start = runner.positions[rid]
            if start + len(toks) > cache.max_pages_per_seq * cache.page_size or \
                    not cache.grow(rid, start, start + len(toks)):
                raise RuntimeError(f"step {rec['step']}: request {rid!r} needs pages for {start + len(toks)} tokens "
                                   f"but the pool of {cache.num_pages} pages (--max-tokens) is exhausted")
            entries.append(StepEntry(rid, toks, list(e.get("want", []))))
        if runner.can_replay(entries):                   # graphs on and a pure decode step
            logits = runner.step_graph(entries).clone()
        else:
            logits = runner.step(entries)
        runner.check_device_status()
        for e in entries:
            cache.advance(e.rid, runner.positions[e.rid], None)
        for rid in rec.get("end", []):
            if cache.holds(rid):
                cache.release(rid)
                runner.end_request(rid)
        return logits


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (rounded up per request to whole pages)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--graphs", action="store_true", help="replay decode steps from CUDA graphs, as generation does")
    a = ap.parse_args(argv)
    if a.page_size < 1 or 64 % a.page_size:
        ap.error("--page-size must divide 64")
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    runner, _ = make_runner(a.model, a.dtype, a.max_tokens, page_size=a.page_size, graphs=a.graphs)
    session = TraceSession(runner)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        logits = session.run_step(rec)
        if logits.shape[0]:
            arr = logits.detach().float().cpu().contiguous().numpy().astype("<f4", copy=False)
            arr.tofile(out / f"{rec['step']}.f32")
        print(f"done {rec['step']}", flush=True)
    return 0
