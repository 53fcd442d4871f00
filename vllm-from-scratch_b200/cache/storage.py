"""Device memory of the cache: one slab of pages per group, one state tensor per
layer execution that keeps state of fixed size.

Layer executions whose mixers need the same thing (number of key/value heads,
head size, window) form a group.  A group's slab is ``[executions, 2, pages,
kv_heads, page_size, head_dim]`` (index 1: 0 = keys, 1 = values), so the keys of
one page and head are ``page_size * head_dim`` contiguous elements: one bulk copy
per page and head for the attention kernels.  The reference allocates ``[2,
pages, page_size, kv_heads, head_dim]`` per layer (minivllm/worker/
kv_cache_alloc.py:65-85); grouping by need follows minivllm/worker/
gpu_model_runner.py:521-580.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import CacheView, KVPagesNeed, StateNeed


@dataclass
class CacheGroup:
    need: KVPagesNeed
    entries: list[int]              # schedule entries that own a slice of the slab
    slab: torch.Tensor


class CacheStorage:
    def __init__(self, needs: list[KVPagesNeed | StateNeed | None], cache_from: list[int | None],
                 page_size: int, num_pages: int, max_requests: int, dtype: torch.dtype,
                 device: torch.device | str) -> None:
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.groups: list[CacheGroup] = []
        self.states: dict[int, torch.Tensor] = {}
        group_of_key: dict[tuple, int] = {}
        owner_view: dict[int, CacheView] = {}
        members: dict[int, list[int]] = {}
        for index, need in enumerate(needs):
            if isinstance(need, KVPagesNeed):
                key = (need.num_kv_heads, need.head_dim, need.window)
                group = group_of_key.setdefault(key, len(group_of_key))
                members.setdefault(group, []).append(index)
        for key, group in sorted(group_of_key.items(), key=lambda item: item[1]):
            need = KVPagesNeed(*key)
            slab = torch.zeros((len(members[group]), 2, num_pages, need.num_kv_heads, page_size,
                                need.head_dim), dtype=dtype, device=device)
            self.groups.append(CacheGroup(need, members[group], slab))
            for position, index in enumerate(members[group]):
                owner_view[index] = CacheView("pages", group, slab[position, 0], slab[position, 1])
        for index, need in enumerate(needs):
            if isinstance(need, StateNeed):
                # one spare row past the last slot: padded rows of fixed-shape batches land there
                state = torch.zeros((max_requests + 1, *need.shape), dtype=need.dtype, device=device)
                self.states[index] = state
                owner_view[index] = CacheView("state", state=state)
        self.views: list[CacheView] = []
        for index, need in enumerate(needs):
            source = cache_from[index]
            if source is not None:
                view = owner_view.get(source)
                if view is None:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {source}, which has none")
                self.views.append(CacheView(view.kind, view.group, view.keys, view.values, view.state,
                                            writable=False))
            else:
                self.views.append(owner_view.get(index, CacheView("none")))

    @staticmethod
    def bytes_per_page(needs: list[KVPagesNeed | StateNeed | None], page_size: int, dtype: torch.dtype) -> int:
        """Memory one page number costs over all executions that own a cache of pages (every
        group's pool has the same number of pages, so a page number exists once in each)."""
        element = torch.empty((), dtype=dtype).element_size()
        return sum(2 * need.num_kv_heads * page_size * need.head_dim * element
                   for need in needs if isinstance(need, KVPagesNeed))

    @property
    def group_windows(self) -> list[int | None]:
        return [group.need.window for group in self.groups]

    @property
    def has_state(self) -> bool:
        return bool(self.states)

    def zero_slots(self, slots: list[int]) -> None:
        """State of a request starts at zero: at admission and after preemption."""
        if slots and self.states:
            for state in self.states.values():
                index = torch.tensor(slots, dtype=torch.long, device=state.device)
                state.index_fill_(0, index, 0)

    def num_bytes(self) -> int:
        total = sum(g.slab.numel() * g.slab.element_size() for g in self.groups)
        return total + sum(s.numel() * s.element_size() for s in self.states.values())

    def bytes_per_token(self) -> int:
        """Cache bytes one position of one request occupies over all groups."""
        return sum(len(g.entries) * 2 * g.need.num_kv_heads * g.need.head_dim * g.slab.element_size()
                   for g in self.groups)
