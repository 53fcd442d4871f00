"""The cache manager: pages for every group of layers, a block table per request
and group, and one resident slot per request for state of fixed size.

A *group* is a set of layer executions with the same need: all keys, or a window
of them.  Each group has a pool of pages of its own (``cache/pool.py``) and its
own block table per request.  Pages come back when a request ends, when it is
preempted, and, in a windowed group, as soon as every position they hold lies
before the window of all positions still to be computed.  The reference has one
group for Qwen3 and frees nothing mid-request (minivllm/core/
single_type_kv_cache_manager.py:180-201); the allocation rule (atomic: all or
nothing), the prefix hashing and the hit cap follow minivllm/core/
kv_cache_manager.py:135-215 and minivllm/core/kv_cache_utils.py:274-341.

This module is host-side bookkeeping only; the tensors live in ``cache/storage.py``.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

from .pool import PagePool

RELEASED = -1


class CacheError(RuntimeError):
    pass


@dataclass
class _Held:
    slot: int
    # Per group: logical page index -> physical page (RELEASED once given back).
    pages: list[list[int]]
    released: list[int]                 # per group: leading pages already given back
    hashes: list[bytes] = field(default_factory=list)   # chained hash of each full page of tokens
    published: int = 0                  # full pages already offered to the prefix cache


class CacheManager:
    def __init__(self, group_windows: list[int | None], page_size: int, num_pages: int,
                 max_requests: int, enable_prefix_caching: bool = False,
                 has_state: bool = False) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        if max_requests <= 0:
            raise ValueError(f"max_requests must be positive, got {max_requests}")
        self.page_size = page_size
        self.group_windows = list(group_windows)
        self.pools = [PagePool(num_pages) for _ in self.group_windows]
        self.max_requests = max_requests
        # A published prefix can stand for a request's past only where every group
        # keeps all keys and no layer keeps state of its own.
        self.prefix_caching = bool(enable_prefix_caching and self.pools and not has_state
                                   and all(w is None for w in self.group_windows))
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._held: dict[str, _Held] = {}
        self._fresh_slots: set[int] = set()

    # -------------------------------------------------------------------- slots
    def admit(self, request_id: str) -> int:
        """Give the request its resident slot (kept until :meth:`release`)."""
        if request_id in self._held:
            raise CacheError(f"request {request_id!r} is already admitted")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._held[request_id] = _Held(slot, [[] for _ in self.pools], [0] * len(self.pools))
        self._fresh_slots.add(slot)
        return slot

    def is_admitted(self, request_id: str) -> bool:
        return request_id in self._held

    def slot(self, request_id: str) -> int:
        return self._held[request_id].slot

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def take_fresh_slots(self) -> list[int]:
        """Slots handed out (or reset) since the last call: their state must be zeroed."""
        fresh, self._fresh_slots = sorted(self._fresh_slots), set()
        return fresh

    # -------------------------------------------------------------------- pages
    def _pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def pages_missing(self, request_id: str, total_tokens: int) -> list[int]:
        held = self._held[request_id]
        return [max(0, self._pages_for(total_tokens) - len(pages)) for pages in held.pages]

    def can_allocate(self, request_id: str, total_tokens: int) -> bool:
        return all(need <= pool.num_free
                   for need, pool in zip(self.pages_missing(request_id, total_tokens), self.pools))

    def allocate(self, request_id: str, total_tokens: int) -> bool:
        """Make the request's block tables cover ``total_tokens`` positions.
        Either every group gets its pages or nothing changes and False is returned."""
        if not self.can_allocate(request_id, total_tokens):
            return False
        held = self._held[request_id]
        for need, pool, pages in zip(self.pages_missing(request_id, total_tokens), self.pools, held.pages):
            pages.extend(pool.take(need))
        return True

    def block_table(self, request_id: str, group: int) -> list[int]:
        return self._held[request_id].pages[group]

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    # ------------------------------------------------------------- prefix cache
    def _chain(self, held: _Held, token_ids, upto_pages: int) -> None:
        size = self.page_size
        while len(held.hashes) < upto_pages:
            index = len(held.hashes)
            digest = hashlib.sha256()
            digest.update(b"page-chain-v1")
            digest.update(held.hashes[-1] if held.hashes else b"\x00" * 32)
            digest.update(b"".join(int(t).to_bytes(8, "little", signed=True)
                                   for t in token_ids[index * size:(index + 1) * size]))
            held.hashes.append(digest.digest())

    def match_prefix(self, request_id: str, token_ids) -> int:
        """Attach already published pages that hold a prefix of ``token_ids`` to a
        request that holds no pages yet.  Returns the number of tokens covered;
        at most ``len(token_ids) - 1``, so that one token is always computed
        (minivllm/core/kv_cache_manager.py:135-150)."""
        held = self._held[request_id]
        if not self.prefix_caching or any(held.pages):
            return 0
        limit = (len(token_ids) - 1) // self.page_size
        self._chain(held, token_ids, limit)
        found: list[list[int]] = []
        for index in range(limit):
            pages = [pool.lookup(held.hashes[index]) for pool in self.pools]
            if any(page is None for page in pages):
                break
            found.append(pages)
        for pages in found:
            for group, page in enumerate(pages):
                self.pools[group].share(page)
                held.pages[group].append(page)
        held.published = len(found)
        return len(found) * self.page_size

    # ------------------------------------------------------------ after a step
    def commit(self, request_id: str, computed_tokens: int, token_ids=None) -> None:
        """Tell the manager that the request's first ``computed_tokens`` positions
        are in the cache.  Windowed groups give back pages no later position can
        read; full pages are offered to the prefix cache (``token_ids`` needed)."""
        held = self._held[request_id]
        for group, window in enumerate(self.group_windows):
            if window is None:
                continue
            # The next query sits at position `computed_tokens` and reads keys from
            # computed_tokens - window + 1 on; pages wholly before that are done.
            first_needed = computed_tokens - window + 1
            done = max(0, first_needed) // self.page_size
            done = min(done, len(held.pages[group]))
            if done > held.released[group]:
                pages = held.pages[group]
                back = [pages[i] for i in range(held.released[group], done)]
                for i in range(held.released[group], done):
                    pages[i] = RELEASED
                self.pools[group].give_back(back)
                held.released[group] = done
        if self.prefix_caching and token_ids is not None:
            full = min(computed_tokens, len(token_ids)) // self.page_size
            self._chain(held, token_ids, full)
            for index in range(held.published, full):
                for group, pool in enumerate(self.pools):
                    pool.publish(held.pages[group][index], held.hashes[index])
            held.published = max(held.published, full)

    def drop_pages(self, request_id: str) -> None:
        """Give back every page of the request but keep its slot (preemption:
        it will be computed again from its first token)."""
        held = self._held[request_id]
        for group, pool in enumerate(self.pools):
            live = [page for page in held.pages[group] if page != RELEASED]
            pool.give_back(list(reversed(live)))       # tail first: evicted before its prefix
            held.pages[group] = []
            held.released[group] = 0
        held.published = 0
        held.hashes = []
        self._fresh_slots.add(held.slot)

    def release(self, request_id: str) -> None:
        """The request is over: pages and slot come back."""
        if request_id not in self._held:
            raise CacheError(f"request {request_id!r} holds nothing (released twice?)")
        self.drop_pages(request_id)
        held = self._held.pop(request_id)
        self._fresh_slots.discard(held.slot)
        self._free_slots.append(held.slot)

    # --------------------------------------------------------------- invariants
    def stats(self) -> dict[str, int]:
        return {
            "requests": len(self._held),
            "free_slots": len(self._free_slots),
            **{f"group{g}_free_pages": pool.num_free for g, pool in enumerate(self.pools)},
            **{f"group{g}_published_pages": pool.num_published for g, pool in enumerate(self.pools)},
        }

    def check_invariants(self) -> None:
        slots = [held.slot for held in self._held.values()] + self._free_slots
        if sorted(slots) != list(range(self.max_requests)):
            raise CacheError(f"slots lost or held twice: {sorted(slots)}")
        for group, pool in enumerate(self.pools):
            holders: dict[int, int] = {}
            for held in self._held.values():
                for page in held.pages[group]:
                    if page != RELEASED:
                        holders[page] = holders.get(page, 0) + 1
            pool.check(holders)
