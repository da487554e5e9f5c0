"""`Engine`: the Python entry point.

    eng = Engine("path/to/model", dtype="bfloat16", max_num_seqs=64, ...)
    outs = eng.generate([[1, 2, 3], [4, 5]], SamplingParams(max_tokens=16))

The constructor's options are those of tzar-beep/Tensorline's `BatchEngine`
(tensorline/batch_engine.py:79-85) where this engine has the feature.  Token ids are the primary
interface; strings are accepted when the model folder has tokenizer files.  tzar-beep/Tensorline
runs its scheduler on a thread of its own and streams text to HTTP handlers
(batch_engine.py:141, :190-227); servers are not part of this engine, so the loop runs in the
caller's thread: `generate` drives `step()` until its requests are done, and `add_request` +
`step()` are public for callers that interleave their own work.
"""
from __future__ import annotations

import itertools
import time
import warnings
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..cache import CacheManager, PagedKV
from ..config.engine import EngineConfig
from ..models import build_model, load_model
from ..parts import Runtime
from ..sampling import GenStats, Sampler, SamplingParams, draw_rows, request_seed
from .runner import ModelRunner, StepEntry
from .scheduler import Request, Scheduler


@dataclass
class Output:
    token_ids: list
    finish_reason: str
    stats: GenStats
    text: str | None = None
    prompt_token_ids: list = field(default_factory=list)


def pick_device(requested: str = "auto") -> torch.device:
    """tensorline/engine.py:18-21, without the CPU: this engine's kernels are CUDA only."""
    if requested in ("auto", "cuda"):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this engine runs on the GPU only")
        return torch.device("cuda", torch.cuda.current_device())
    dev = torch.device(requested)
    if dev.type != "cuda":
        raise RuntimeError(f"device {requested!r}: this engine runs on the GPU only")
    return dev


class Engine:
    def __init__(self, model, device: str = "auto", dtype: str = "auto", *, weights: dict | None = None,
                 tokenizer=None, **options):
        """`model`: a model folder, or a typed configuration together with `weights`
        (name -> tensor, already on the device) for models that never touch a disk."""
        self.options = EngineConfig(dtype=dtype, **options)
        self.options.validate()
        self.device = pick_device(device)
        act = {"bfloat16": torch.bfloat16, "float32": torch.float32}[self.options.resolved_dtype()]
        self.rt = Runtime(self.device, act, self.options.block_size)
        if weights is None:
            self.model_dir = Path(model)
            self.model, self.config = load_model(self.model_dir, self.rt)
        else:
            self.model_dir = None
            self.config = model
            self.model = build_model(model, self.rt)
            self.model.bind(weights)
        self.tokenizer = tokenizer
        if self.options.max_model_len > (self.model.spec.max_position_embeddings or self.options.max_model_len):
            self.options.max_model_len = self.model.spec.max_position_embeddings
        o = self.options
        needs = self.model.cache_needs()
        num_blocks = o.num_blocks
        if num_blocks is None:                                       # tensorline/batch_engine.py:89-97
            per_page = sum(2 * n.num_kv_heads * n.head_dim * o.block_size * act.itemsize
                           for n in needs.values() if isinstance(n, PagedKV)) or 1
            if o.kv_cache_gb is not None:
                num_blocks = int(o.kv_cache_gb * (1 << 30)) // per_page
            else:
                free, _ = torch.cuda.mem_get_info(self.device)
                num_blocks = int(free * o.kv_mem_fraction) // per_page
            num_blocks = max(1, min(num_blocks, o.max_num_seqs * -(-o.max_model_len // o.block_size)))
        if num_blocks * o.block_size < o.max_num_seqs * 256:         # tensorline/batch_engine.py:98-102
            warnings.warn(f"KV cache holds only {num_blocks * o.block_size} tokens ({num_blocks} pages): "
                          f"{o.max_num_seqs} concurrent sequences will queue or preempt.", stacklevel=2)
        self.cache = CacheManager(needs, page_size=o.block_size, num_pages=num_blocks, max_num_seqs=o.max_num_seqs,
                                  max_model_len=o.max_model_len, prefix_caching=o.prefix_caching)
        self.runner = ModelRunner(self.model, self.cache)
        self.runner.use_graphs = bool(o.cuda_graphs)
        self.scheduler = Scheduler(self.cache, max_num_seqs=o.max_num_seqs, max_batched_tokens=o.max_batched_tokens,
                                   max_model_len=o.max_model_len)
        self.sampler = Sampler(self.device)
        self._ids = itertools.count()
        eos = self.model.spec.eos_token_id
        self.default_stops = {eos} if eos is not None else set()     # tensorline/engine.py:76-77
        self._known_to_runner: set = set()
        # Overlap (tensorline/batch_engine.py:478-533): in steady decoding the next step is launched from the
        # tokens still on the device before the previous step's tokens are read back.
        self.overlap = bool(o.overlap and o.cuda_graphs)
        self._inflight = None                            # (requests, DecodeHandle) of the step not yet read back
        self.overlapped_steps = 0

    # ------------------------------------------------------------------ requests
    def _encode(self, prompt):
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass token ids or a tokenizer")
            return list(self.tokenizer(prompt).input_ids)
        return [int(t) for t in prompt]

    def add_request(self, prompt, params: SamplingParams | None = None) -> Request:
        params = params or SamplingParams()
        ids = self._encode(prompt)
        stops = set() if params.ignore_eos else (set(params.stop_token_ids) or set(self.default_stops))
        req = Request(next(self._ids), len(ids), ids, params, stops, GenStats(), time.perf_counter())
        req.seed = request_seed(self.options.seed, req.rid, params)
        self.scheduler.add(req)
        return req

    def abort(self, req: Request) -> None:
        self.scheduler.abort(req)       # a step in flight for it finishes on the device; its token is dropped
        self._sync_runner()

    def _sync_runner(self) -> None:
        """Tell the runner which requests entered or left the cache since the last step."""
        for rid in [r for r in self._known_to_runner if not self.cache.holds(r)]:
            self.runner.end_request(rid)
            self._known_to_runner.discard(rid)

    # ------------------------------------------------------------------ overlap
    def _launch(self, reqs, prev=None):
        """Start a decode step for `reqs` without waiting for its tokens."""
        entries = [StepEntry(r.rid, [r.tokens[-1] if prev is None else 0], [0]) for r in reqs]
        ahead = 0 if prev is None else 1                 # the step in flight has one token of each request still to come
        draw = draw_rows([(r.params, r.seed, r.num_generated + ahead) for r in reqs])
        handle = self.runner.launch_decode(entries, None if prev is None else prev[1], draw)
        self.scheduler.computed([(r, 1) for r in reqs])
        return reqs, handle

    def _resolve(self, inflight) -> list:
        """Read a launched step's tokens back and accept them; a request that finished one step
        earlier has produced one token too many, which is dropped (tensorline/batch_engine.py:500-508)."""
        reqs, handle = inflight
        toks = self.runner.read_tokens(handle)
        now = time.perf_counter()
        out = []
        for req, tok in zip(reqs, toks):
            if not req.done and self.scheduler.accept(req, tok, now):
                out.append((req, tok))
        self._sync_runner()
        return out

    def _can_continue(self) -> bool:
        """Whether the step after the one in flight can be launched before that one is read back
        (tensorline/batch_engine.py:510-521): same requests, nobody near a limit, a page for one more
        token each.  tzar-beep/Tensorline also asks for greedy requests; here sampled ones go on as well:
        a draw's uniform number depends on (seed, token index) only, so it is known a step ahead, and the
        sampling kernel runs on the device behind the decode graph."""
        reqs = self._inflight[0]
        sch = self.scheduler
        if sch.waiting or len(sch.running) != len(reqs) or any(a is not b for a, b in zip(sch.running, reqs)):
            return False
        for r in reqs:      # the pending token is appended when the step is read back; leave room for one more
            if r.done or r.num_generated + 2 > r.params.max_tokens or len(r.tokens) + 2 > sch.max_model_len:
                return False
        return all(self.cache.grow(r.rid, r.num_computed, r.num_computed + 1) for r in reqs)

    def flush(self) -> list:
        """Read back the step in flight, if any."""
        if self._inflight is None:
            return []
        prev, self._inflight = self._inflight, None
        return self._resolve(prev)

    # ------------------------------------------------------------------ one iteration
    def step(self) -> list:
        """Schedule, run one batch, sample, finish.  Returns [(request, token)] for the tokens that
        became known in this call (with overlap on, a decode step's tokens arrive one call later)."""
        sch = self.scheduler
        try:
            if self._inflight is not None:
                if self._can_continue():
                    prev = self._inflight
                    self._inflight = self._launch(prev[0], prev)
                    self.overlapped_steps += 1
                    return self._resolve(prev)
                return self.flush()
            plan = sch.schedule()
            self._sync_runner()
            if not plan:
                return []
            entries = []
            for req, n in plan:
                if req.rid not in self._known_to_runner or self.runner.positions.get(req.rid) != req.num_computed:
                    self.runner.start_request(req.rid, req.num_computed)      # new, or back after a preemption
                    self._known_to_runner.add(req.rid)
                end = req.num_computed + n
                want = [n - 1] if end == len(req.tokens) else []      # tensorline/batch_engine.py:376
                entries.append(StepEntry(req.rid, req.tokens[req.num_computed:end], want))
            if self.overlap and self.runner.can_replay(entries):
                self._inflight = self._launch([r for r, _ in plan])      # its tokens are read at the next call
                return []
            sampled = [req for (req, n), e in zip(plan, entries) if e.want]
            rows = [(r.params, r.seed, r.num_generated) for r in sampled]
            tokens = self.runner.step_and_sample(entries, self.sampler, rows)
            sch.computed(plan)
            now = time.perf_counter()
            out = []
            for req, tok in zip(sampled, tokens):
                if sch.accept(req, tok, now):
                    out.append((req, tok))
            self._sync_runner()
            return out
        except Exception as e:                                       # tensorline/batch_engine.py:568-576
            self._inflight = None
            sch.fail_all(e)
            self._sync_runner()
            raise

    def generate(self, prompts, params: SamplingParams | list | None = None) -> list:
        """Run the prompts to completion; returns one `Output` per prompt, in order."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        plist = params if isinstance(params, list) else [params] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while any(not r.done for r in reqs):
            self.step()
        outs = []
        for r in reqs:
            if r.error is not None:
                raise r.error
            text = self.tokenizer.decode(r.output_tokens, skip_special_tokens=True) if self.tokenizer else None
            outs.append(Output(r.output_tokens, r.stats.finish_reason, r.stats, text, r.tokens[:r.prompt_len]))
        return outs

    def render_chat(self, messages: list) -> str:
        """Chat messages as one prompt string (tensorline/engine.py:79-84): the tokenizer's template
        if it has one, else "role: content" lines."""
        if self.tokenizer is not None and getattr(self.tokenizer, "chat_template", None):
            return self.tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)
        return "".join(f"{m['role']}: {m['content']}\n" for m in messages) + "assistant:"

    def shutdown(self) -> None:
        """Fail what is still queued and drop the device tensors (tensorline/batch_engine.py:144-157)."""
        self.scheduler.fail_all(RuntimeError("engine shut down"))
        self._sync_runner()
        self.runner = self.model = None

    # ------------------------------------------------------------------ figures
    def stats(self) -> dict:
        s = self.scheduler
        return {"steps": s.steps, "preemptions": s.preemptions, "max_running_seen": s.max_running_seen,
                "prompt_tokens_total": s.prompt_tokens_total, "prefix_hit_tokens": s.prefix_hit_tokens,
                "requests_finished": dict(s.finished), "free_pages": self.cache.num_free_pages(),
                "num_pages": self.cache.num_pages, "graph_replays": getattr(self.runner, "graph_replays", 0),
                "overlapped_steps": self.overlapped_steps}
