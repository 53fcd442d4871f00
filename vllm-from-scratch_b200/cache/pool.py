"""One pool of pages: who holds each page, which are free, which still carry a
published prefix.

Behaviour follows the reference's block pool (minivllm/core/block_pool.py:31-182,
minivllm/core/kv_cache_utils.py:121-271): a reference count per page; a free
queue from whose head pages are taken; a page that comes back without a published
hash goes to the head (used again first), one with a hash to the tail (evicted
last, still hittable until it is handed out again).  The queue here is an ordered
dictionary, which gives the same O(1) removal from the middle as the reference's
linked list.
"""

from __future__ import annotations

from collections import OrderedDict


class PagePoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self.ref_count = [0] * num_pages
        self._free: OrderedDict[int, None] = OrderedDict((page, None) for page in range(num_pages))
        self._hash_of_page: dict[int, bytes] = {}
        self._page_of_hash: dict[bytes, int] = {}

    # ------------------------------------------------------------------ queries
    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_published(self) -> int:
        return len(self._hash_of_page)

    def lookup(self, digest: bytes) -> int | None:
        return self._page_of_hash.get(digest)

    # ------------------------------------------------------------------ changes
    def take(self, count: int) -> list[int]:
        """``count`` pages from the head of the free queue, each with one holder."""
        if count > len(self._free):
            raise PagePoolError(f"asked for {count} pages, {len(self._free)} are free")
        pages = []
        for _ in range(count):
            page, _ = self._free.popitem(last=False)
            digest = self._hash_of_page.pop(page, None)
            if digest is not None and self._page_of_hash.get(digest) == page:
                del self._page_of_hash[digest]
            self.ref_count[page] = 1
            pages.append(page)
        return pages

    def share(self, page: int) -> None:
        """One more holder of a published page (a prefix hit)."""
        if self.ref_count[page] == 0:
            if page not in self._free:
                raise PagePoolError(f"page {page} has no holder and is not in the free queue")
            del self._free[page]
        self.ref_count[page] += 1

    def give_back(self, pages: list[int]) -> None:
        """Drop one holder of each page, in the given order."""
        for page in pages:
            if self.ref_count[page] <= 0:
                raise PagePoolError(f"page {page} given back more often than taken")
            self.ref_count[page] -= 1
            if self.ref_count[page] == 0:
                self._free[page] = None
                if page not in self._hash_of_page:
                    self._free.move_to_end(page, last=False)

    def publish(self, page: int, digest: bytes) -> None:
        if page in self._hash_of_page:
            return
        self._hash_of_page[page] = digest
        self._page_of_hash.setdefault(digest, page)

    def forget_published(self) -> None:
        """Drop every published hash (pages keep their holders)."""
        self._hash_of_page.clear()
        self._page_of_hash.clear()

    # --------------------------------------------------------------- invariants
    def check(self, holders: dict[int, int]) -> None:
        """``holders``: page -> number of requests that list it.  Raises if the
        pool's books disagree: a page lost, held twice, or free while held."""
        for page in range(self.num_pages):
            held = holders.get(page, 0)
            if self.ref_count[page] != held:
                raise PagePoolError(f"page {page}: count {self.ref_count[page]}, listed by {held} requests")
            if (page in self._free) != (held == 0):
                raise PagePoolError(f"page {page}: free={page in self._free} with {held} holders")
        for digest, page in self._page_of_hash.items():
            if self._hash_of_page.get(page) != digest:
                raise PagePoolError(f"published hash points at page {page}, which carries another")
