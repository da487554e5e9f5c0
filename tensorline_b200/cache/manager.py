"""`CacheManager`: pages, block tables and fixed-size state slots for all live requests.

What a layer's mixer keeps between steps is declared as a `CacheNeed`:

* `PagedKV(num_kv_heads, head_dim, window)`: keys and values in pages of `page_size` tokens.
  Layers whose needs have the same give-back rule (all keys, or a window of W keys) form one
  *group*; a group has its own page pool and its own block table per request, because a window
  group returns the pages a window has passed while a full group keeps them.
* `SlotState(shape, dtype)`: a tensor of fixed size per request, held in the request's *slot*
  (a small integer given at admission and returned when the request ends, is preempted or is
  aborted).  The slot also indexes the block-table rows.  The Qwen2 decoder has no such state;
  the slots exist for mixers that do.

Everything here is host bookkeeping (numpy tables, Python lists); the device tensors that the
tables and slots index are allocated by the model runner from `groups` and `state_needs`.

Rules kept from tzar-beep/Tensorline: position p of a request lives in page
`table[p // page_size]` at offset `p % page_size` (tensorline/paged.py:202); allocation is
all-or-nothing (paged.py:57-69, batch_engine.py:248-259); only full, fully computed pages are
published for sharing (batch_engine.py:282-290); a fully cached prompt gives back its last
page so that its last token is computed for logits (batch_engine.py:277-279); one extra page
past the pool is a sink for padding rows (paged.py:125-127).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .pages import CacheError, PagePool, page_hash


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of `num_kv_heads` heads of `head_dim`, all of them (`window` None) or
    the last `window` positions."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None

    @property
    def group_key(self):
        return ("paged_kv", self.window)


@dataclass(frozen=True)
class SlotState:
    """Per-request state of fixed size: one tensor of `shape` per slot."""
    shape: tuple
    dtype: str = "float32"

    @property
    def group_key(self):
        return ("slot_state",)


@dataclass
class PageGroup:
    index: int
    window: int | None
    pool: PagePool
    caches: list = field(default_factory=list)          # ids of the cache entries that use this group
    table: np.ndarray | None = None                     # [max_slots + 1, max_pages_per_seq] int32
    version: int = 0                                    # bumped at every write to `table`

    @property
    def scratch_page(self) -> int:
        return self.pool.num_pages


@dataclass
class _Held:
    slot: int
    pages: list                                         # per group: list of page ids, -1 once given back
    hashes: list = field(default_factory=list)          # hashes of the published full pages (full-attention only)


class CacheManager:
    def __init__(self, needs: dict, *, page_size: int, num_pages: int, max_num_seqs: int,
                 max_model_len: int, prefix_caching: bool = True):
        """`needs`: cache id -> `PagedKV` | `SlotState` (one id per cache that a run entry owns)."""
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_pages_per_seq = -(-max_model_len // page_size)
        self.needs = dict(needs)
        self.groups: list[PageGroup] = []
        self.group_of: dict = {}                         # cache id -> group index (paged caches only)
        self.state_needs: dict = {}                      # cache id -> SlotState
        by_key: dict = {}
        for cid, need in self.needs.items():
            if isinstance(need, SlotState):
                self.state_needs[cid] = need
                continue
            if not isinstance(need, PagedKV):
                raise TypeError(f"cache {cid!r}: unknown need {need!r}")
            if need.window is not None and need.window < 1:
                raise ValueError(f"cache {cid!r}: window must be positive")
            g = by_key.get(need.group_key)
            if g is None:
                g = PageGroup(len(self.groups), need.window, PagePool(num_pages, False))
                g.table = np.full((max_num_seqs + 1, self.max_pages_per_seq), num_pages, dtype=np.int32)
                by_key[need.group_key] = g
                self.groups.append(g)
            g.caches.append(cid)
            self.group_of[cid] = g.index
        # Sharing a prefix needs every cache of a request to be restorable from pages alone.
        self.prefix_caching = bool(prefix_caching and len(self.groups) == 1
                                   and self.groups[0].window is None and not self.state_needs)
        for g in self.groups:
            g.pool.prefix_caching = self.prefix_caching
        self._free_slots = list(range(max_num_seqs - 1, -1, -1))
        self._held: dict = {}
        self.padding_slot = max_num_seqs                 # its table rows point at the scratch pages
        # Called before any write to a group's table: the owner of a device copy that may still be
        # in flight from this memory waits for it here.
        self.before_table_write = None

    def _touch(self, g: PageGroup) -> None:
        if self.before_table_write is not None:
            self.before_table_write()
        g.version += 1

    # ------------------------------------------------------------------ figures
    @property
    def num_pages(self) -> int:
        return self.groups[0].pool.num_pages if self.groups else 0

    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def can_ever_hold(self, num_tokens: int) -> bool:
        """Whether a request of `num_tokens` tokens could lie in an otherwise empty cache."""
        for g in self.groups:
            live = num_tokens if g.window is None else min(num_tokens, g.window + self.page_size)
            if -(-live // self.page_size) > g.pool.num_pages:
                return False
        return True

    def slot(self, rid) -> int:
        return self._held[rid].slot

    def holds(self, rid) -> bool:
        return rid in self._held

    def pages(self, rid, group: int = 0) -> list[int]:
        return list(self._held[rid].pages[group])

    # ------------------------------------------------------------------ life of a request
    def admit(self, rid, tokens=None) -> int | None:
        """Give `rid` a slot and, if sharing is on, the published pages of the longest prefix
        of `tokens`.  Returns the number of tokens whose cache is already there, or None if no
        slot is free (tensorline/batch_engine.py:266-280)."""
        if rid in self._held:
            raise CacheError(f"request {rid!r} is already admitted")
        if not self._free_slots:
            return None
        held = _Held(self._free_slots.pop(), [[] for _ in self.groups])
        self._held[rid] = held
        cached = 0
        if self.prefix_caching and tokens is not None:
            ps, pool, parent = self.page_size, self.groups[0].pool, None
            pages = held.pages[0]
            for i in range(len(tokens) // ps):
                chunk = tokens[i * ps:(i + 1) * ps]
                h = page_hash(parent, chunk)
                page = pool.lookup(h, parent, chunk)
                if page is None:
                    break
                pages.append(page)
                held.hashes.append(h)
                parent = h
            if pages and len(pages) * ps == len(tokens):       # fully cached: recompute the last page
                pool.free([pages.pop()])
                held.hashes.pop()
            cached = len(pages) * ps
            self._write_table(0, held.slot, 0, pages)
        return cached

    def _first_needed_page(self, g: PageGroup, start: int) -> int:
        """Index of the first page a query at position >= `start` can still read."""
        if g.window is None:
            return 0
        return max(0, start - g.window + 1) // self.page_size

    def grow(self, rid, start: int, upto: int) -> bool:
        """Make room for positions [start, upto): first give back what every window has passed
        (keys before `start - window + 1`), then take the missing pages of every group, all or
        nothing (tensorline/batch_engine.py:248-259)."""
        held = self._held[rid]
        if upto > self.max_pages_per_seq * self.page_size:
            raise CacheError(f"request {rid!r} would hold {upto} tokens; tables end at "
                             f"{self.max_pages_per_seq * self.page_size}")
        self._release_behind_window(held, start)
        want = -(-upto // self.page_size)
        need = [max(0, want - len(p)) for p in held.pages]
        if any(n > g.pool.num_free for n, g in zip(need, self.groups)):
            return False
        for g, n, pages in zip(self.groups, need, held.pages):
            if n:
                got = g.pool.allocate(n)
                first = len(pages)
                pages += got
                self._write_table(g.index, held.slot, first, got)
        return True

    def _release_behind_window(self, held: _Held, start: int) -> None:
        for g, pages in zip(self.groups, held.pages):
            if g.window is None:
                continue
            first = min(self._first_needed_page(g, start), len(pages))
            gone = [(i, p) for i, p in enumerate(pages[:first]) if p >= 0]
            if gone:
                g.pool.free([p for _, p in gone])
                self._touch(g)
                for i, _ in gone:
                    pages[i] = -1
                    g.table[held.slot, i] = g.scratch_page

    def advance(self, rid, num_computed: int, tokens) -> None:
        """After a step: publish the pages that are now full and computed
        (tensorline/batch_engine.py:282-290) and give back pages behind every window."""
        held = self._held[rid]
        self._release_behind_window(held, num_computed)
        if not self.prefix_caching:
            return
        ps, pool, pages = self.page_size, self.groups[0].pool, held.pages[0]
        while len(held.hashes) < min(num_computed, len(tokens)) // ps:
            i = len(held.hashes)
            parent = held.hashes[-1] if i else None
            chunk = tokens[i * ps:(i + 1) * ps]
            h = page_hash(parent, chunk)
            held.hashes.append(h)
            pool.register(pages[i], h, parent, chunk)

    def release(self, rid) -> None:
        """Give back everything `rid` holds: pages of every group and its slot
        (tensorline/batch_engine.py:261-264, :358-367)."""
        held = self._held.pop(rid, None)
        if held is None:
            raise CacheError(f"request {rid!r} released but not admitted (double release)")
        for g, pages in zip(self.groups, held.pages):
            g.pool.free([p for p in pages if p >= 0])
            self._touch(g)
            g.table[held.slot, :] = g.scratch_page
        self._free_slots.append(held.slot)

    def _write_table(self, group: int, slot: int, first: int, pages) -> None:
        if pages:
            self._touch(self.groups[group])
            self.groups[group].table[slot, first:first + len(pages)] = pages

    # ------------------------------------------------------------------ self check (tests)
    def check(self) -> None:
        """No page lost, held twice without a count for it, or freed twice; no slot lost."""
        slots = [h.slot for h in self._held.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a slot is held twice or both held and free")
        if len(slots) + len(self._free_slots) != self.max_num_seqs:
            raise CacheError("a slot is lost")
        for g in self.groups:
            counts: dict = {}
            for h in self._held.values():
                for p in h.pages[g.index]:
                    if p >= 0:
                        counts[p] = counts.get(p, 0) + 1
            g.pool.check(counts)
            for h in self._held.values():
                row = g.table[h.slot]
                for i, p in enumerate(h.pages[g.index]):
                    if row[i] != (p if p >= 0 else g.scratch_page):
                        raise CacheError(f"table row of slot {h.slot} disagrees with the page list at {i}")
