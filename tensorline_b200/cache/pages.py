"""`PagePool`: the host-side owner of one group's fixed-size cache pages.

Pages are reference counted.  A page whose count drops to zero goes to the tail of a
least-recently-freed list but keeps its contents and, if it was published, its content hash;
a later request with the same prefix takes it back instead of recomputing it, and it is evicted
only when `allocate` needs the room.  The behaviour follows `BlockAllocator` of
tzar-beep/Tensorline (tensorline/paged.py:28-93); the differences are explicit errors in place
of an assert (paged.py:75), a 64-bit chained hash of our own in place of Python's `hash`
(paged.py:96-97), and the hashed tokens kept with the page so that a hit is verified.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict


class CacheError(RuntimeError):
    """A page or slot was freed twice, freed without being held, or the pool is corrupt."""


def page_hash(parent: int | None, tokens) -> int:
    """Hash of one full page of token ids chained over everything before it
    (tensorline/paged.py:96-97)."""
    h = hashlib.blake2b(digest_size=8)
    h.update(struct.pack("<q", -1 if parent is None else parent & 0x7FFFFFFFFFFFFFFF))
    h.update(struct.pack(f"<{len(tokens)}i", *tokens))
    return int.from_bytes(h.digest(), "little") & 0x7FFFFFFFFFFFFFFF


class PagePool:
    def __init__(self, num_pages: int, prefix_caching: bool = True):
        if num_pages < 1:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self.prefix_caching = prefix_caching
        self._free: OrderedDict[int, None] = OrderedDict.fromkeys(range(num_pages))   # oldest first
        self._ref = [0] * num_pages
        self._hash_of: list[int | None] = [None] * num_pages
        self._key_of: list[tuple | None] = [None] * num_pages       # (parent hash, tokens) of a published page
        self._cached: dict[int, int] = {}                            # content hash -> page

    # ---- figures
    @property
    def num_free(self) -> int:
        """Pages nobody holds, evictable cached ones included (tensorline/paged.py:48-51)."""
        return len(self._free)

    @property
    def num_cached(self) -> int:
        return len(self._cached)

    def refcount(self, page: int) -> int:
        return self._ref[page]

    # ---- allocation
    def allocate(self, n: int) -> list[int] | None:
        """`n` pages or nothing (tensorline/paged.py:57-69): least recently freed first; a page
        taken from the list loses its published contents."""
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            return None
        out = []
        for _ in range(n):
            page, _ = self._free.popitem(last=False)
            h = self._hash_of[page]
            if h is not None:
                del self._cached[h]
                self._hash_of[page] = None
                self._key_of[page] = None
            self._ref[page] = 1
            out.append(page)
        return out

    def free(self, pages) -> None:
        """Drop one reference on each page.  The pages of a request's tail are the least likely
        to be shared, so they enter the list first and are evicted first
        (tensorline/paged.py:71-77)."""
        for page in reversed(list(pages)):
            if not 0 <= page < self.num_pages:
                raise CacheError(f"page {page} is outside the pool of {self.num_pages}")
            if self._ref[page] <= 0:
                raise CacheError(f"page {page} freed while nobody holds it (double free)")
            self._ref[page] -= 1
            if self._ref[page] == 0:
                self._free[page] = None

    # ---- prefix sharing
    def lookup(self, h: int, parent: int | None = None, tokens=None) -> int | None:
        """Take a reference on the published page with hash `h` (tensorline/paged.py:79-87).
        If `tokens` is given, the page's recorded tokens must equal them."""
        page = self._cached.get(h) if self.prefix_caching else None
        if page is None:
            return None
        if tokens is not None and self._key_of[page] != (parent, tuple(tokens)):
            return None                                      # a 64-bit collision: treat as a miss
        if self._ref[page] == 0:
            del self._free[page]
        self._ref[page] += 1
        return page

    def register(self, page: int, h: int, parent: int | None = None, tokens=None) -> None:
        """Publish a fully computed page under its hash unless that hash is already published
        (tensorline/paged.py:89-93)."""
        if not self.prefix_caching or h in self._cached:
            return
        if self._ref[page] <= 0:
            raise CacheError(f"page {page} published while nobody holds it")
        if self._hash_of[page] is not None:
            return
        self._cached[h] = page
        self._hash_of[page] = h
        self._key_of[page] = (parent, tuple(tokens)) if tokens is not None else None

    # ---- self check (tests)
    def check(self, held: dict[int, int] | None = None) -> None:
        """Raise unless every page is either in the free list with count 0 or held with a
        positive count; `held` (page -> expected count) is compared if given."""
        for page in range(self.num_pages):
            in_free = page in self._free
            if in_free and self._ref[page] != 0:
                raise CacheError(f"page {page} is in the free list with count {self._ref[page]}")
            if not in_free and self._ref[page] <= 0:
                raise CacheError(f"page {page} is lost: not free and count {self._ref[page]}")
        for h, page in self._cached.items():
            if self._hash_of[page] != h:
                raise CacheError(f"page {page} and hash table disagree")
        if held is not None:
            for page in range(self.num_pages):
                if self._ref[page] != held.get(page, 0):
                    raise CacheError(f"page {page}: count {self._ref[page]}, holders say {held.get(page, 0)}")
