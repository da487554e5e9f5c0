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
published for sharing (batch_engine.py:282-290); a prompt found whole in the cache still computes
its last token, for the logits (batch_engine.py:277-279); one extra page past the pool is a sink
for padding rows (paged.py:125-127).  Beyond it: every page group shares prefixes, a window group
too (a new request takes only the published pages its window still reaches, the entries before
them point at the sink); groups may have pools of different sizes.
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
    pages: list                                         # per group: page ids in position order, -1 once given back
    digests: list = field(default_factory=list)         # chained digests of the request's full, computed pages
    offered: list = field(default_factory=list)         # per group: how many of them were offered for publishing


class CacheManager:
    def __init__(self, needs: dict, *, page_size: int, num_pages, max_num_seqs: int,
                 max_model_len: int, prefix_caching: bool = True):
        """`needs`: cache id -> `PagedKV` | `SlotState` (one id per cache that a run entry owns).
        `num_pages`: pages of every group's pool, or {window (None: all keys): pages} per group."""
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
                n = num_pages[need.window] if isinstance(num_pages, dict) else num_pages
                g = PageGroup(len(self.groups), need.window, PagePool(n, False))
                g.table = np.full((max_num_seqs + 1, self.max_pages_per_seq), n, dtype=np.int32)
                by_key[need.group_key] = g
                self.groups.append(g)
            g.caches.append(cid)
            self.group_of[cid] = g.index
        # A shared prefix is restored from pages alone: every page group can do that (a window group
        # needs only the pages its window still reaches), state of fixed size cannot.
        self.prefix_caching = bool(prefix_caching and self.groups and not self.state_needs)
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

    def capacity(self, rid) -> int:
        """Positions [0, capacity) of `rid` have a table entry in every group (a page, or the sink for
        what a window has passed); a step may not write at or beyond it.  Without page groups there
        is no bound."""
        held = self._held[rid]
        if not self.groups:
            return self.max_model_len
        return min(len(p) for p in held.pages) * self.page_size

    def room_for(self, rid, start: int) -> int:
        """How many tokens from position `start` on `grow` could make room for right now, counting the
        pages the request already holds, the idle ones and those its windows have passed at `start`."""
        held = self._held[rid]
        room = self.max_pages_per_seq * self.page_size - start
        for g, pages in zip(self.groups, held.pages):
            first = self._first_needed_page(g, start)
            # a passed page that others share comes back to nobody: count the request's own only
            returning = sum(1 for p in pages[:first] if p >= 0 and g.pool.refcount(p) == 1)
            room = min(room, (len(pages) + g.pool.num_free + returning) * self.page_size - start)
        return max(0, room)

    # ------------------------------------------------------------------ life of a request
    def _chain(self, tokens, upto_pages: int, known: list) -> list:
        """Chained digests of the first `upto_pages` full pages of `tokens`, extending `known`."""
        ps = self.page_size
        for i in range(len(known), upto_pages):
            known.append(page_hash(known[-1] if known else None, tokens[i * ps:(i + 1) * ps]))
        return known

    def _shared_prefix_pages(self, tokens) -> tuple:
        """(k, digests): the largest number k of leading full pages of `tokens` that every group can
        serve from published pages.  A group that keeps all keys needs all k pages; a window group
        only those a query at position k * page_size can still read.  At least one token is left to
        compute (tensorline/batch_engine.py:277-279: the last token's logits are wanted)."""
        ps = self.page_size
        most = (len(tokens) - 1) // ps
        digests = self._chain(tokens, most, [])

        def served(g: PageGroup, i: int) -> bool:
            return g.pool.find(digests[i], digests[i - 1] if i else None, tokens[i * ps:(i + 1) * ps]) is not None

        for g in self.groups:                            # groups that keep everything bound k from above
            if g.window is None:
                k = 0
                while k < most and served(g, k):
                    k += 1
                most = k
        for k in range(most, 0, -1):
            if all(served(g, i) for g in self.groups if g.window is not None
                   for i in range(self._first_needed_page(g, k * ps), k)):
                return k, digests[:k]
        return 0, []

    def admit(self, rid, tokens=None) -> int | None:
        """Give `rid` a slot and, if sharing is on, the published pages of the longest prefix of
        `tokens` that all groups can serve.  Returns the number of tokens whose cache is already
        there, or None if no slot is free."""
        if rid in self._held:
            raise CacheError(f"request {rid!r} is already admitted")
        if not self._free_slots:
            return None
        held = _Held(self._free_slots.pop(), [[] for _ in self.groups], offered=[0] * len(self.groups))
        self._held[rid] = held
        if not self.prefix_caching or tokens is None:
            return 0
        ps = self.page_size
        k, digests = self._shared_prefix_pages(tokens)
        if k == 0:
            return 0
        held.digests = digests
        for g, pages in zip(self.groups, held.pages):
            first = self._first_needed_page(g, k * ps)
            pages += [-1] * first                        # what the window has passed is never read
            for i in range(first, k):
                page = g.pool.adopt(digests[i], digests[i - 1] if i else None, tokens[i * ps:(i + 1) * ps])
                if page is None:
                    raise CacheError(f"published page {i} of group {g.index} vanished during admission")
                pages.append(page)
            held.offered[g.index] = k
            self._write_table(g.index, held.slot, first, pages[first:])
        return k * ps

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
                got = g.pool.take(n)
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
                g.pool.drop([p for _, p in gone])
                self._touch(g)
                for i, _ in gone:
                    pages[i] = -1
                    g.table[held.slot, i] = g.scratch_page

    def advance(self, rid, num_computed: int, tokens) -> None:
        """After a step: offer the pages that are now full and computed for sharing, in every group
        that still holds them (only full pages whose tokens are all computed:
        tensorline/batch_engine.py:282-290), then give back the pages behind every window."""
        held = self._held[rid]
        if self.prefix_caching and tokens is not None:
            ps = self.page_size
            full = min(num_computed, len(tokens)) // ps
            digests = self._chain(tokens, full, held.digests)
            for g, pages in zip(self.groups, held.pages):
                for i in range(held.offered[g.index], full):
                    if pages[i] >= 0:
                        g.pool.publish(pages[i], digests[i], digests[i - 1] if i else None, tokens[i * ps:(i + 1) * ps])
                held.offered[g.index] = max(held.offered[g.index], full)
        self._release_behind_window(held, num_computed)

    def release(self, rid) -> None:
        """Give back everything `rid` holds: pages of every group and its slot
        (tensorline/batch_engine.py:261-264, :358-367)."""
        held = self._held.pop(rid, None)
        if held is None:
            raise CacheError(f"request {rid!r} released but not admitted (double release)")
        for g, pages in zip(self.groups, held.pages):
            g.pool.drop([p for p in pages if p >= 0])
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
