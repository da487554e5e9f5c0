"""`PagePool`: who holds which cache page of one group, on the host.

The rules are those of tzar-beep/Tensorline's block allocator (tensorline/paged.py:28-93):

* a page has a number of holders; a page without holders is *idle*: it keeps its contents and, if
  it was published under a content digest, stays findable, until `take` needs the room
  (paged.py:71-77, :79-87);
* `take(n)` is all-or-nothing and uses up the pages that have been idle longest (paged.py:57-69);
* a request's later pages are less likely to be shared than its earlier ones, so when a request
  lets go of a run of pages the last of the run becomes the first to be used up (paged.py:72-73);
* a digest is published once; a second page with the same contents stays private (paged.py:89-93);
* letting go of a page nobody holds is an error (an assert at paged.py:75; an exception here).

The state is a handful of flat arrays indexed by page number, not containers of page objects: the
holder counts, the links of an intrusive ring that threads the idle pages from the longest idle to
the most recently idle (so joining, leaving and reviving are O(1) without searching), the published
digest, an *epoch* that counts how often the page's contents were given up (a holder that remembers
(page, epoch) can tell a recycled page from the one it knew), and, for published pages, the token
ids and the parent digest they were published with: a hit on a digest is accepted only if those
agree, where tzar-beep/Tensorline trusts Python's `hash` (paged.py:96-97).
"""
from __future__ import annotations

import hashlib

import numpy as np


class CacheError(RuntimeError):
    """A page or slot was let go twice or without being held, or the bookkeeping is inconsistent."""


_NO_DIGEST = 0


def page_hash(parent: int | None, tokens) -> int:
    """Digest of one full page of token ids, chained over everything before it (the idea of
    tensorline/paged.py:96-97 with a 63-bit BLAKE2 digest; never 0, which means "not published")."""
    h = hashlib.blake2b(digest_size=8)
    h.update(int(parent or 0).to_bytes(8, "little"))
    h.update(np.asarray(tokens, dtype="<i4").tobytes())
    return (int.from_bytes(h.digest(), "little") >> 1) or 1


class PagePool:
    def __init__(self, num_pages: int, prefix_caching: bool = True):
        if num_pages < 1:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        n = self.num_pages = int(num_pages)
        self.prefix_caching = bool(prefix_caching)
        self._holders = np.zeros(n, dtype=np.int32)
        # The idle ring: entry n is the anchor; `_after[n]` is the page that has been idle longest.
        self._after = np.arange(1, n + 2, dtype=np.int64)
        self._before = np.arange(-1, n, dtype=np.int64)
        self._after[n], self._before[0] = 0, n
        self._idle = n
        self._epoch = np.zeros(n, dtype=np.int64)
        self._digest = np.zeros(n, dtype=np.int64)
        self._parent = np.zeros(n, dtype=np.int64)
        self._tokens: list = [None] * n                  # token ids a published page was published with
        self._published: dict = {}                       # digest -> page

    # ---- figures
    @property
    def num_free(self) -> int:
        """Pages without a holder, published ones included (tensorline/paged.py:48-51)."""
        return self._idle

    @property
    def num_cached(self) -> int:
        return len(self._published)

    def refcount(self, page: int) -> int:
        return int(self._holders[page])

    def epoch(self, page: int) -> int:
        return int(self._epoch[page])

    # ---- the idle ring
    def _leave_ring(self, page: int) -> None:
        b, a = self._before[page], self._after[page]
        self._after[b], self._before[a] = a, b
        self._idle -= 1

    def _join_ring(self, page: int) -> None:
        anchor = self.num_pages
        last = self._before[anchor]
        self._after[last], self._before[page] = page, last
        self._after[page], self._before[anchor] = anchor, page
        self._idle += 1

    def _forget(self, page: int) -> None:
        d = int(self._digest[page])
        if d != _NO_DIGEST:
            del self._published[d]
            self._digest[page] = _NO_DIGEST
            self._tokens[page] = None
        self._epoch[page] += 1

    # ---- taking and letting go
    def take(self, n: int) -> list | None:
        """`n` pages with one holder each, or None and no change.  The longest idle pages go
        first; what they had published is forgotten."""
        if n < 0:
            raise ValueError("negative page count")
        if n > self._idle:
            return None
        got = []
        for _ in range(n):
            page = int(self._after[self.num_pages])
            self._leave_ring(page)
            self._forget(page)
            self._holders[page] = 1
            got.append(page)
        return got

    def drop(self, pages) -> None:
        """One holder less on each page of a request's run `pages` (in the request's order)."""
        run = [int(p) for p in pages]
        for page in run:
            if not 0 <= page < self.num_pages:
                raise CacheError(f"page {page} is outside the pool of {self.num_pages}")
        for page in run[::-1]:                           # the end of the run is used up first
            if self._holders[page] < 1:
                raise CacheError(f"page {page} let go while nobody holds it (double free)")
            self._holders[page] -= 1
            if self._holders[page] == 0:
                self._join_ring(page)

    # ---- sharing by content
    def find(self, digest: int, parent: int | None = None, tokens=None) -> int | None:
        """The page published under `digest`, or None; no holder is added.  With `tokens` the hit
        counts only if the page was published with these tokens and this parent digest."""
        if not self.prefix_caching:
            return None
        page = self._published.get(int(digest))
        if page is None:
            return None
        if tokens is not None:
            known = self._tokens[page]
            if known is None or int(self._parent[page]) != int(parent or 0) or \
                    not np.array_equal(known, np.asarray(tokens, dtype=np.int32)):
                return None                              # another text with the same digest
        return page

    def adopt(self, digest: int, parent: int | None = None, tokens=None) -> int | None:
        """`find`, and the caller becomes one more holder of the page; an idle page is revived."""
        page = self.find(digest, parent, tokens)
        if page is None:
            return None
        if self._holders[page] == 0:
            self._leave_ring(page)
        self._holders[page] += 1
        return page

    def publish(self, page: int, digest: int, parent: int | None = None, tokens=None) -> bool:
        """Publish a held, fully written page; False if the digest or the page is already published."""
        digest = int(digest)
        if not self.prefix_caching or digest in self._published:
            return False
        if self._holders[page] < 1:
            raise CacheError(f"page {page} published while nobody holds it")
        if self._digest[page] != _NO_DIGEST:
            return False
        self._published[digest] = int(page)
        self._digest[page] = digest
        self._parent[page] = int(parent or 0)
        self._tokens[page] = None if tokens is None else np.array(tokens, dtype=np.int32)
        return True

    # ---- self check (tests)
    def check(self, held: dict | None = None) -> None:
        """Raise unless the ring holds exactly the pages without holders, every published digest
        points at a page that knows it, and (if given) `held` (page -> holders) matches."""
        n = self.num_pages
        seen, page = set(), int(self._after[n])
        while page != n:
            if page in seen or len(seen) > n:
                raise CacheError("the idle ring is broken")
            if int(self._before[int(self._after[page])]) != page:
                raise CacheError(f"the idle ring's links disagree at page {page}")
            seen.add(page)
            page = int(self._after[page])
        if len(seen) != self._idle:
            raise CacheError(f"{self._idle} pages counted idle, {len(seen)} in the ring")
        for page in range(n):
            c = int(self._holders[page])
            if (page in seen) != (c == 0):
                raise CacheError(f"page {page} is lost or idle while held: {c} holders, "
                                 f"{'in' if page in seen else 'not in'} the ring")
        for d, page in self._published.items():
            if int(self._digest[page]) != d:
                raise CacheError(f"page {page} and the published digests disagree")
        if held is not None:
            for page in range(n):
                if int(self._holders[page]) != held.get(page, 0):
                    raise CacheError(f"page {page}: {int(self._holders[page])} holders, the requests say "
                                     f"{held.get(page, 0)}")
