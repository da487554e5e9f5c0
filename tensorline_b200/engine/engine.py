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
from .scheduler import Request, Scheduler, Slice


@dataclass
class Output:
    token_ids: list
    finish_reason: str
    stats: GenStats
    text: str | None = None
    prompt_token_ids: list = field(default_factory=list)


@dataclass
class _StepInFlight:
    """A decode step that is on the device while the host goes on: its requests, in row order, and the
    runner's handle for its tokens."""
    requests: list
    handle: object


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
        # Running ahead (the idea of tensorline/batch_engine.py:478-533): while the same requests keep
        # decoding, the next step is started from the tokens still on the device before the host has
        # seen the previous step's tokens.  At most one step is ahead of the host.
        self.overlap = bool(o.overlap and o.cuda_graphs)
        self._ahead: _StepInFlight | None = None
        self.overlapped_steps = 0
        self.last_step_kind = "idle"                     # what the last step() held: "decode", "prompt", "mixed" or "idle"

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
        """Tell the runner which requests left the cache since the last step."""
        for rid in [r for r in self._known_to_runner if not self.cache.holds(r)]:
            self.runner.end_request(rid)
            self._known_to_runner.discard(rid)

    # ------------------------------------------------------------------ decode steps that run ahead of the host
    def _start_decode(self, reqs, after: "_StepInFlight | None" = None) -> "_StepInFlight":
        """Put a decode step for `reqs` on the device and return without its tokens.  `after`: the step
        of the same requests that is still in flight; its tokens, on the device, are this step's inputs."""
        behind = 0 if after is None else 1               # tokens of each request the host has not seen yet
        entries = [StepEntry(r.rid, [r.tokens[-1] if after is None else 0], [0]) for r in reqs]
        draw = draw_rows([(r.params, r.seed, r.num_generated + behind) for r in reqs])
        handle = self.runner.launch_decode(entries, None if after is None else after.handle, draw)
        self.scheduler.computed([Slice(r, r.num_computed, 1) for r in reqs])
        return _StepInFlight(list(reqs), handle)

    def _collect(self, step: "_StepInFlight") -> list:
        """Wait for a started step, check the device status that came back with it, and hand its tokens
        to the scheduler.  A request that ended with the step before has produced one token too many,
        which is dropped (tensorline/batch_engine.py:500-508)."""
        toks = self.runner.read_tokens(step.handle)      # raises KernelError if a kernel gave up on a wait
        now = time.perf_counter()
        kept = [(req, tok) for req, tok in zip(step.requests, toks)
                if not req.done and self.scheduler.accept(req, tok, now)]
        self._sync_runner()
        return kept

    def _may_run_ahead(self, step: "_StepInFlight") -> bool:
        """Whether the step after `step` can be started before `step` is read: nothing waits, the running
        set is exactly `step`'s requests, each has room for two more tokens under its limits, and the
        cache has a place for one more token each (tensorline/batch_engine.py:510-521).
        tzar-beep/Tensorline also asks for greedy requests; here sampled ones go on as well: a draw's
        uniform number depends on (seed, token index) only, so it is known a step ahead, and the sampling
        kernel runs on the device behind the decode graph."""
        sch = self.scheduler
        if sch.waiting or len(sch.running) != len(step.requests):
            return False
        for mine, theirs in zip(step.requests, sch.running):
            if mine is not theirs or mine.done:
                return False
            if mine.num_generated + 2 > mine.params.max_tokens or len(mine.tokens) + 2 > sch.max_model_len:
                return False
        return all(self.cache.grow(r.rid, r.num_computed, r.num_computed + 1) for r in step.requests)

    def flush(self) -> list:
        """Read back the step in flight, if any."""
        if self._ahead is None:
            return []
        step, self._ahead = self._ahead, None
        return self._collect(step)

    # ------------------------------------------------------------------ one iteration
    def step(self) -> list:
        """Schedule, run one batch, sample, finish.  Returns [(request, token)] for the tokens that
        became known in this call (with overlap on, a decode step's tokens arrive one call later)."""
        try:
            if self._ahead is not None:
                if not self._may_run_ahead(self._ahead):
                    self.last_step_kind = "idle"         # only reads the step in flight back
                    return self.flush()
                earlier = self._ahead
                self._ahead = self._start_decode(earlier.requests, after=earlier)
                self.overlapped_steps += 1
                self.last_step_kind = "decode"
                return self._collect(earlier)
            return self._scheduled_step()
        except Exception as e:                           # tensorline/batch_engine.py:568-576
            self._ahead = None
            self.scheduler.fail_all(e)
            self._sync_runner()
            raise

    def _scheduled_step(self) -> list:
        sch = self.scheduler
        plan = sch.schedule()
        self._sync_runner()
        ones, rest = plan.kinds()
        self.last_step_kind = "idle" if not plan else "decode" if not rest else "prompt" if not ones else "mixed"
        if not plan:
            return []
        entries = []
        for sl in plan:
            rid = sl.request.rid
            if rid not in self._known_to_runner or self.runner.positions.get(rid) != sl.start:
                self.runner.start_request(rid, sl.start)             # new, or back after a preemption
                self._known_to_runner.add(rid)
            entries.append(StepEntry(rid, sl.tokens, [sl.count - 1] if sl.wants_logits else []))
        if self.overlap and self.runner.can_replay(entries):
            self._ahead = self._start_decode([sl.request for sl in plan])     # its tokens are read at the next call
            return []
        sampled = [sl.request for sl in plan if sl.wants_logits]
        rows = [(r.params, r.seed, r.num_generated) for r in sampled]
        tokens = self.runner.step_and_sample(entries, self.sampler, rows)
        self.runner.check_device_status()
        sch.computed(plan)
        now = time.perf_counter()
        kept = [(req, tok) for req, tok in zip(sampled, tokens) if sch.accept(req, tok, now)]
        self._sync_runner()
        return kept

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
