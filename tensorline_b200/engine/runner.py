"""`ModelRunner`: the one step function.

    runner.step([StepEntry(rid, tokens, want), ...]) -> logits [wanted, vocab] float32

A step takes, for each request in it, that request's next tokens: a portion of its prompt of any
length, cut anywhere, or a single decoded token; all entries run as ONE flattened batch
(tensorline/paged.py:190-207).  The step computes only the tokens it is given: keys and values of
earlier tokens come from the cache pages that earlier steps wrote.  It returns the logits at the
wanted places (`want`: indices into the entry's tokens), in entry order
(tensorline/paged.py:278-287, which returns the last row only).

The runner owns the device side of the cache: the page tensors of every cache-owning run entry,
the per-slot state tensors, and device copies of the block tables; the `CacheManager` owns the
bookkeeping.  A request's position is tracked here (`positions[rid]`), so an entry needs no
`start` (tensorline/paged.py:100-106 passes it explicitly).

Steps that hold only single decoded tokens can be replayed from a CUDA graph, one graph per
batch-size bucket (tensorline/cuda_graphs.py:38-126); tables and lengths are read from device
memory, so there are no buckets over context length.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import CacheManager, PagedKV, SlotState
from ..models.spec import Model
from ..parts import KVCacheView, Runtime, StateView
from .. import ops


@dataclass
class StepEntry:
    rid: object
    tokens: list
    want: list = field(default_factory=list)       # places among `tokens` whose logits are returned


@dataclass
class StepContext:
    """Device-side description of one step, handed to every part."""
    T: int
    B: int
    ids: torch.Tensor                   # int32 [T]
    pos: torch.Tensor                   # int32 [T] absolute position of each token in its request
    req_slot: torch.Tensor              # int32 [T] slot of the request that owns each token
    q_start: torch.Tensor               # int32 [B + 1] first row of each request's tokens
    start_pos: torch.Tensor             # int32 [B] position of each request's first token of the step
    slots: torch.Tensor                 # int32 [B]
    want_rows: torch.Tensor             # int32 [R]
    tables: list                        # per page group: int32 [slots + 1, max pages]
    page_size: int
    decode_only: bool                   # every request brings exactly one token
    max_q_len: int
    max_ctx: int                        # largest position + 1 in the step
    h_q_start: list                     # host copies for parts written in Python
    h_start_pos: list
    h_slots: list
    force_exact_attention: bool = False
    graph_max_ctx: int = 0              # > 0: the step is captured in a graph; size for this context
    scratch: dict = field(default_factory=dict)    # per-step scratch of kernels, keyed by name


_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
           "int32": torch.int32, "int64": torch.int64}


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, *, device=None):
        self.model = model
        self.cache = cache
        self.rt: Runtime = model.rt
        self.device = torch.device(device) if device is not None else self.rt.device
        if self.device.type != "cuda":
            raise RuntimeError("ModelRunner needs a CUDA device: this engine has no CPU path")
        self.page_size = cache.page_size
        self.positions: dict = {}       # rid -> number of tokens already in the cache
        self.force_exact_attention = False
        needs = model.cache_needs()
        self.caches: dict = {}
        for cid, need in needs.items():
            if isinstance(need, PagedKV):
                g = cache.group_of[cid]
                shape = (cache.groups[g].pool.num_pages + 1, need.num_kv_heads, self.page_size, need.head_dim)
                self.caches[cid] = KVCacheView(torch.zeros(shape, dtype=self.rt.act_dtype, device=self.device),
                                               torch.zeros(shape, dtype=self.rt.act_dtype, device=self.device), g)
            elif isinstance(need, SlotState):
                shape = (cache.max_num_seqs + 1,) + tuple(need.shape)
                self.caches[cid] = StateView(torch.zeros(shape, dtype=_DTYPES[need.dtype], device=self.device))
        # The manager's tables move into pinned memory (it writes them in place), so that the copy
        # to the device before each step is one asynchronous transfer per group.
        self._host_tables = []
        for g in cache.groups:
            pinned = torch.from_numpy(g.table.copy()).pin_memory()
            g.table = pinned.numpy()
            self._host_tables.append(pinned)
        self.tables = [t.to(self.device) for t in self._host_tables]
        self._table_versions = [g.version for g in cache.groups]
        self._table_event = None
        cache.before_table_write = self._wait_for_table_copy
        self.vocab_size = model.spec.vocab_size
        self.use_graphs = False
        self.graph_replays = 0
        self._graphs: dict = {}
        self._graph_pool = None
        # State of fixed size lives at fixed addresses indexed by slot (padding rows use the spare row), so a
        # model with such state is captured like any other, as long as its parts read the step from device
        # tensors only (`Part.graph_capturable`).
        self._graphable = model.graph_capturable()
        self._token_hosts = [torch.zeros(cache.max_num_seqs + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._flip = 0
        # temperature, top-p and uniform number per row for steps that sample on the device without waiting
        self._draw_hosts = [torch.zeros(3, cache.max_num_seqs, dtype=torch.float32).pin_memory() for _ in range(4)]
        self._draw_events = [None] * 4
        self._draw_turn = 0
        self._draw_dev = torch.zeros(3, cache.max_num_seqs, dtype=torch.float32, device=self.device)

    def _wait_for_table_copy(self) -> None:
        if self._table_event is not None:
            self._table_event.synchronize()
            self._table_event = None

    def _sync_tables(self) -> None:
        """Copy the block tables that changed since the last step to the device."""
        copied = False
        for i, g in enumerate(self.cache.groups):
            if self._table_versions[i] != g.version:
                self.tables[i].copy_(self._host_tables[i], non_blocking=True)
                self._table_versions[i] = g.version
                copied = True
        if copied:
            self._table_event = torch.cuda.Event()
            self._table_event.record()

    # ------------------------------------------------------------------ bytes
    def cache_bytes_per_token(self) -> int:
        total = 0
        for c in self.caches.values():
            if isinstance(c, KVCacheView):
                total += 2 * c.k.shape[1] * c.k.shape[3] * c.k.element_size()
        return total

    # ------------------------------------------------------------------ requests
    def start_request(self, rid, cached_tokens: int = 0) -> None:
        """A request enters (or re-enters after preemption) with `cached_tokens` of its tokens
        already in shared pages.  State slots start from zero."""
        self.positions[rid] = cached_tokens
        slot = self.cache.slot(rid)
        for c in self.caches.values():
            if isinstance(c, StateView):
                c.state[slot].zero_()

    def end_request(self, rid) -> None:
        self.positions.pop(rid, None)

    # ------------------------------------------------------------------ the step
    def build_context(self, entries) -> StepContext:
        """The step's description, packed on the host into one int32 array and copied to the device in one transfer:
        per token its id, position and request slot; per request its first row, first position and slot; the wanted rows."""
        B = len(entries)
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=B)
        if B and int(lens.min()) < 1:
            bad = entries[int(lens.argmin())]
            raise ValueError(f"request {bad.rid!r}: an entry needs at least one token")
        q_start = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(lens, out=q_start[1:])
        T = int(q_start[-1])
        start_pos = np.fromiter((self.positions[e.rid] for e in entries), dtype=np.int64, count=B)
        slots = np.fromiter((self.cache.slot(e.rid) for e in entries), dtype=np.int64, count=B)
        want_rows = []
        for i, e in enumerate(entries):
            room = self.cache.capacity(e.rid)
            if start_pos[i] + lens[i] > room:
                raise RuntimeError(f"request {e.rid!r}: positions up to {start_pos[i] + lens[i]} but pages for {room}; "
                                   "grow its cache before the step")
            for w in e.want:
                if not 0 <= w < lens[i]:
                    raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {lens[i]} tokens")
                want_rows.append(int(q_start[i]) + w)
        R = len(want_rows)
        packed = np.empty(3 * T + 3 * B + 1 + R, dtype=np.int32)
        cut = np.cumsum([0, T, T, T, B + 1, B, B, R])
        for i, e in enumerate(entries):
            packed[q_start[i]:q_start[i + 1]] = e.tokens
        ids = packed[:T]
        if T and (int(ids.min()) < 0 or int(ids.max()) >= self.vocab_size):
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        row_of = np.repeat(np.arange(B), lens)
        packed[cut[1]:cut[2]] = start_pos[row_of] + (np.arange(T) - q_start[row_of])
        packed[cut[2]:cut[3]] = slots[row_of]
        packed[cut[3]:cut[4]] = q_start
        packed[cut[4]:cut[5]] = start_pos
        packed[cut[5]:cut[6]] = slots
        packed[cut[6]:cut[7]] = want_rows
        dev = torch.from_numpy(packed).to(self.device, non_blocking=False)
        parts = [dev[cut[i]:cut[i + 1]] for i in range(7)]
        self._sync_tables()
        ends = start_pos + lens
        return StepContext(T=T, B=B, ids=parts[0], pos=parts[1], req_slot=parts[2], q_start=parts[3],
                           start_pos=parts[4], slots=parts[5], want_rows=parts[6], tables=self.tables,
                           page_size=self.page_size, decode_only=bool(B) and int(lens.max()) == 1, max_q_len=int(lens.max()) if B else 0,
                           max_ctx=int(ends.max()) if B else 0, h_q_start=q_start.tolist(), h_start_pos=start_pos.tolist(),
                           h_slots=slots.tolist(), force_exact_attention=self.force_exact_attention)

    @torch.inference_mode()
    def step(self, entries) -> torch.Tensor:
        """Run one batch; returns logits [number of wanted places, vocab], float32, on the device."""
        entries = list(entries)
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
        ctx = self.build_context(entries)
        logits = self.model.forward(ctx, self.caches)
        for e in entries:
            self.positions[e.rid] += len(e.tokens)
        return logits

    def step_and_sample(self, entries, sampler, rows) -> list:
        """One step followed by one sampled token per wanted place; `rows` as `Sampler.sample`.
        A step of single decoded tokens that all want their logits replays a CUDA graph; if all of
        them are greedy the argmax is part of the graph and only the tokens come back."""
        entries = list(entries)
        if self._can_replay(entries):
            g = self._run_graph(entries)
            n = len(entries)
            if all(p.temperature <= 0 for p, _, _ in rows):
                got = g.tokens.tolist()
                if got[-1] != 0:
                    ops.raise_device_status(self.device, got[-1])
                return got[:n]
            return sampler.sample(g.logits[:n], rows)
        logits = self.step(entries)
        return sampler.sample(logits, rows)

    # ------------------------------------------------------------------ CUDA-graph decode
    def _can_replay(self, entries) -> bool:
        return (self.use_graphs and self._graphable and 0 < len(entries) <= self.cache.max_num_seqs
                and all(len(e.tokens) == 1 and list(e.want) == [0] and self.positions[e.rid] > 0 for e in entries))

    def _bucket(self, n: int) -> int:
        """Batch sizes 1, 2, 4, ... and the sequence limit itself (tensorline/cuda_graphs.py:30-35)."""
        b = 1
        while b < n:
            b *= 2
        return min(b, self.cache.max_num_seqs)

    def _capture(self, nb: int):
        dev = self.device
        buf = torch.zeros(7 * nb + 1, dtype=torch.int32, device=dev)
        host = torch.zeros(7 * nb + 1, dtype=torch.int32).pin_memory()
        cut = np.cumsum([0, nb, nb, nb, nb + 1, nb, nb, nb])
        parts = [buf[cut[i]:cut[i + 1]] for i in range(7)]
        pad = self.cache.padding_slot
        host[2 * nb:3 * nb] = pad                                  # req_slot
        host[3 * nb:4 * nb + 1] = torch.arange(nb + 1, dtype=torch.int32)   # q_start: one token each
        host[5 * nb + 1:6 * nb + 1] = pad                          # slots
        host[6 * nb + 1:7 * nb + 1] = torch.arange(nb, dtype=torch.int32)   # every row's logits
        buf.copy_(host)
        ctx = StepContext(T=nb, B=nb, ids=parts[0], pos=parts[1], req_slot=parts[2], q_start=parts[3],
                          start_pos=parts[4], slots=parts[5], want_rows=parts[6], tables=self.tables,
                          page_size=self.page_size, decode_only=True, max_q_len=1, max_ctx=self.cache.max_model_len,
                          h_q_start=list(range(nb + 1)), h_start_pos=[0] * nb, h_slots=[pad] * nb,
                          force_exact_attention=self.force_exact_attention, graph_max_ctx=self.cache.max_model_len)
        tokens = torch.zeros(nb + 1, dtype=torch.int32, device=dev)     # the rows' tokens, then the device status word
        status = ops.device_status(dev)

        def run():
            logits = self.model.forward(ctx, self.caches)
            ops.argmax(logits, tokens[:nb])
            tokens[nb:].copy_(status[:1])                    # a wait that ran out inside a kernel travels with the tokens
            return logits

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                              # warm-up outside the capture: lazy
            for _ in range(2):                                     # library handles, workspaces, kernel attributes
                run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        # Nothing may free device memory while the stream is capturing: collect garbage (graphs and
        # pools of engines that are gone) now, and keep the collector off until the capture ends.
        gc.collect()
        torch.cuda.synchronize()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            before, counts = ops.launch_count(), ops.kernel_counts.copy()
            with torch.cuda.graph(graph, pool=self._graph_pool, capture_error_mode="thread_local"):
                logits = run()
            per_replay = ops.launch_count() - before
            kernels = dict(ops.kernel_counts - counts)
        finally:
            if gc_was_on:
                gc.enable()
        hosts = [host] + [host.clone().pin_memory() for _ in range(3)]
        g = _DecodeGraph(graph, buf, hosts, [None] * len(hosts), logits, tokens, nb, launches=per_replay, kernels=kernels)
        self._graphs[nb] = g
        return g

    # ------------------------------------------------------------------ decode without waiting for the tokens
    def can_replay(self, entries) -> bool:
        return self._can_replay(list(entries))

    def graph_kernels(self, batch: int) -> dict:
        """Kernel variants inside the decode graph that serves `batch` requests: name -> calls per replay
        (captures the graph if it does not exist yet)."""
        nb = self._bucket(batch)
        return dict((self._graphs.get(nb) or self._capture(nb)).kernels)

    def step_graph(self, entries) -> torch.Tensor:
        """`step` for entries that `can_replay`: the same batch through the captured decode graph of its
        batch-size bucket.  Returns the logits [len(entries), vocab] as a view of the graph's output buffer
        (valid until the next replay of that bucket)."""
        entries = list(entries)
        if not self._can_replay(entries):
            raise ValueError("step_graph takes single tokens of running requests that all want their logits, "
                             "with graphs switched on")
        return self._run_graph(entries).logits[:len(entries)]

    @torch.inference_mode()
    def launch_decode(self, entries, ids_from=None, draw=None):
        """Replay the decode graph for `entries` and start copying its tokens to the host without waiting
        (tensorline/batch_engine.py:478-498).  `ids_from`: the handle of the previous launch of the same
        requests in the same order; its tokens, still on the device, are this step's input ids.  `draw`:
        None (every row takes the graph's argmax) or (temperatures, top-p values, uniform numbers) per row:
        the sampling kernel then runs behind the graph and its tokens take the place of the argmax."""
        entries = list(entries)
        n = len(entries)
        g = self._run_graph(entries, None if ids_from is None else ids_from.graph.tokens[:n])
        if draw is not None:
            turn = self._draw_turn = (self._draw_turn + 1) % len(self._draw_hosts)
            if self._draw_events[turn] is not None:
                self._draw_events[turn].synchronize()
            host = self._draw_hosts[turn]
            host[:, :n] = torch.tensor(draw, dtype=torch.float32)
            self._draw_dev.copy_(host, non_blocking=True)
            self._draw_events[turn] = torch.cuda.Event()
            self._draw_events[turn].record()
            d = self._draw_dev
            ops.sample(g.logits[:n], d[0, :n], d[1, :n], d[2, :n], g.tokens[:n])
        self._flip ^= 1
        host = self._token_hosts[self._flip][:g.batch + 1]
        host.copy_(g.tokens, non_blocking=True)              # one copy: the bucket's tokens and the status word
        ev = torch.cuda.Event()
        ev.record()
        return DecodeHandle(g, n, host, ev)

    def read_tokens(self, handle) -> list:
        """The tokens of a launched step, once it has finished.  Raises `KernelError` if a kernel of the
        step (or of an earlier one) gave up on a wait: its output is not valid."""
        handle.event.synchronize()
        got = handle.host.tolist()
        if got[-1] != 0:
            ops.raise_device_status(self.device, got[-1])
        return got[:handle.n]

    def check_device_status(self) -> None:
        """After an eager step whose results the host has already waited for: raise `KernelError` if a
        kernel gave up on a wait (a synchronising read of one word; a no-op for engines whose kernels
        have no such waits)."""
        ops.check_device_status(self.device)

    @torch.inference_mode()
    def _run_graph(self, entries, dev_ids=None):
        n = len(entries)
        nb = self._bucket(n)
        g = self._graphs.get(nb) or self._capture(nb)
        turn = g.turn = (g.turn + 1) % len(g.hosts)          # staging buffers take turns, so that the host
        if g.events[turn] is not None:                       # may prepare a step while earlier ones still run
            g.events[turn].synchronize()
        h = g.hosts[turn].numpy()
        pad = self.cache.padding_slot
        h[0:nb] = 0
        h[nb:2 * nb] = 0
        h[2 * nb:3 * nb] = pad
        h[4 * nb + 1:5 * nb + 1] = 0
        h[5 * nb + 1:6 * nb + 1] = pad
        for i, e in enumerate(entries):
            p = self.positions[e.rid]
            slot = self.cache.slot(e.rid)
            if p + 1 > self.cache.capacity(e.rid):
                raise RuntimeError(f"request {e.rid!r}: no page for position {p}; grow its cache before the step")
            h[i] = e.tokens[0]
            h[nb + i] = p
            h[2 * nb + i] = slot
            h[4 * nb + 1 + i] = p
            h[5 * nb + 1 + i] = slot
        g.buf.copy_(g.hosts[turn], non_blocking=True)
        g.events[turn] = torch.cuda.Event()
        g.events[turn].record()
        if dev_ids is not None:                              # the previous step's tokens, never seen by the host
            g.buf[:n].copy_(dev_ids)
        self._sync_tables()
        g.graph.replay()
        ops.count_launches(g.launches)
        self.graph_replays += 1
        for e in entries:
            self.positions[e.rid] += 1
        return g


@dataclass
class DecodeHandle:
    """A decode step in flight: its graph, batch size, the pinned copy of its tokens and the event after it."""
    graph: object
    n: int
    host: torch.Tensor
    event: object


@dataclass
class _DecodeGraph:
    graph: object
    buf: torch.Tensor
    hosts: list                         # pinned staging buffers of the step's inputs
    events: list                        # per staging buffer: its last copy to the device
    logits: torch.Tensor
    tokens: torch.Tensor
    batch: int
    turn: int = 0
    launches: int = 0                   # kernels of this package inside one replay
    kernels: dict = field(default_factory=dict)         # the same by kernel variant: name -> calls
