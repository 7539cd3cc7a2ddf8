"""The cache manager: pages with a block table per request, and fixed-size state slots.

Cache slots of the model's schedule are sorted into *groups*.  Slots whose mixers
keep the same thing (same kv heads, head size and window) share one group: one
pool of page ids, one block table per request, and one tensor
``[slots_in_group, num_pages, 2, kv_heads, page_size, head_dim]`` (2 = keys,
values), so that a page id addresses the same tokens in every layer of the group.
Groups with different needs have pools of their own.  A group with a window gives
a page back as soon as every position on it lies behind the window of the
request's next token; all pages go back when the request ends.  Nothing is cleared
on reuse: kernels read only positions below the request's length.

Beside the pages every live request holds one *state slot*, an index into
``[max_requests + 1, *shape]`` tensors of the cache slots whose mixers keep state of
fixed size.  Such state is zeroed when the slot is handed to a new request.

The reference keeps one contiguous buffer per sequence, sized for ``--max-seq``
tokens (src/inference.cu:146-148), and clears it wholesale (src/inference.cu:174-176).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import torch

from ..parts.base import FixedStateSpec, PagedKVSpec
from .pages import IdPool, OutOfPages

RELEASED = -1            # block-table entry of a page that a window has passed


@dataclass
class PagedKVView:
    """What a paged mixer sees of its cache slot during one step."""
    pages: Optional[torch.Tensor]        # [num_pages, 2, kv_heads, page_size, head_dim]
    block_table: Optional[torch.Tensor]  # [requests, blocks] int32, RELEASED where passed
    page_size: int
    writes: bool


@dataclass
class StateView:
    """What a mixer with fixed-size state sees of its cache slot during one step."""
    state: Optional[torch.Tensor]        # [max_requests, *shape]
    slots: Optional[torch.Tensor]        # [requests] int32: the state slot of each request
    writes: bool


class _PagedGroup:
    def __init__(self, spec: PagedKVSpec, page_size: int, num_pages: int):
        self.spec = spec
        self.page_size = page_size
        self.pool = IdPool(num_pages, "page")
        self.cache_slots: list[int] = []
        self.tables: dict[Hashable, list[int]] = {}
        self.storage: Optional[torch.Tensor] = None

    def blocks_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def new_pages_needed(self, req, new_length: int) -> int:
        return max(0, self.blocks_for(new_length) - len(self.tables.get(req, ())))

    def first_needed_block(self, length: int) -> int:
        """Index of the first block the token at position ``length`` may still read."""
        if self.spec.window is None:
            return 0
        return max(0, length - self.spec.window + 1) // self.page_size


class CacheManager:
    def __init__(self, cache_specs: Sequence[PagedKVSpec | FixedStateSpec | None], *,
                 page_size: int, num_pages: int, max_requests: int,
                 kv_dtype: torch.dtype = torch.bfloat16, device=None):
        if page_size < 1:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.kv_dtype = kv_dtype
        self.device = device
        self.groups: list[_PagedGroup] = []
        self._slot_group: dict[int, tuple[int, int]] = {}      # cache slot -> (group, index in group)
        self._state_specs: dict[int, FixedStateSpec] = {}
        self._state_storage: dict[int, torch.Tensor] = {}
        by_spec: dict[PagedKVSpec, int] = {}
        for slot, spec in enumerate(cache_specs):
            if isinstance(spec, PagedKVSpec):
                if spec not in by_spec:
                    by_spec[spec] = len(self.groups)
                    self.groups.append(_PagedGroup(spec, page_size, num_pages))
                g = by_spec[spec]
                self._slot_group[slot] = (g, len(self.groups[g].cache_slots))
                self.groups[g].cache_slots.append(slot)
            elif isinstance(spec, FixedStateSpec):
                self._state_specs[slot] = spec
            elif spec is not None:
                raise TypeError(f"cache slot {slot}: unknown cache spec {spec!r}")
        self.null_page = num_pages
        self.state_slots = IdPool(max_requests, "state slot")
        self._lengths: dict[Hashable, int] = {}
        self._state_slot: dict[Hashable, int] = {}
        self._version: dict[Hashable, int] = {}
        self._versions = 0
        if device is not None:
            for g in self.groups:
                s = g.spec
                # one page more than the pool hands out: ``null_page``, where padding rows of a
                # fixed-size (graph) batch write and read without touching a request's pages
                g.storage = torch.zeros(
                    (len(g.cache_slots), num_pages + 1, 2, s.num_kv_heads, page_size, s.head_dim),
                    dtype=kv_dtype, device=device)
            for slot, spec in self._state_specs.items():
                # one slot more than requests can hold, for padding rows
                self._state_storage[slot] = torch.zeros(
                    (max_requests + 1, *spec.shape), dtype=spec.dtype, device=device)

    # ---- requests ------------------------------------------------------------------------
    def add_request(self, req: Hashable) -> None:
        if req in self._lengths:
            raise KeyError(f"request {req!r} is already live")
        slot = self.state_slots.take()
        self._lengths[req] = 0
        self._state_slot[req] = slot
        self._touch(req)
        for g in self.groups:
            g.tables[req] = []
        for t in self._state_storage.values():
            t[slot].zero_()

    def _touch(self, req: Hashable) -> None:
        self._versions += 1
        self._version[req] = self._versions

    def table_version(self, req: Hashable) -> int:
        """A number that changes whenever the request's block tables change otherwise than by
        gaining entries at their end (the request is new, or a window has passed some pages):
        who mirrors the tables elsewhere copies only the new entries while it stays the same."""
        return self._version[req]

    def has_request(self, req: Hashable) -> bool:
        return req in self._lengths

    def live_requests(self) -> list:
        return list(self._lengths)

    def length(self, req: Hashable) -> int:
        return self._lengths[req]

    def state_slot(self, req: Hashable) -> int:
        return self._state_slot[req]

    def pages_needed(self, req: Hashable, num_tokens: int) -> list[int]:
        """New pages each group must hand out before ``num_tokens`` more tokens fit
        (a request that is not live yet counts from length 0)."""
        new_len = self._lengths.get(req, 0) + num_tokens
        return [g.new_pages_needed(req, new_len) for g in self.groups]

    def can_append(self, req: Hashable, num_tokens: int) -> bool:
        return all(n <= g.pool.num_free
                   for n, g in zip(self.pages_needed(req, num_tokens), self.groups))

    def append(self, req: Hashable, num_tokens: int) -> int:
        """Reserve room for ``num_tokens`` more tokens; all groups or none.  Returns the start position."""
        if num_tokens < 1:
            raise ValueError("append needs at least one token")
        need = self.pages_needed(req, num_tokens)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(
                    f"request {req!r} needs {n} more pages of {g.spec}, {g.pool.num_free} are free")
        for n, g in zip(need, self.groups):
            g.tables[req].extend(g.pool.take() for _ in range(n))
        start = self._lengths[req]
        self._lengths[req] = start + num_tokens
        return start

    def reserve_step(self, items: Sequence[tuple[Hashable, int]],
                     max_position: Optional[int] = None) -> list[int]:
        """Make room for one step: ``items`` are (request, number of new tokens).  Requests
        that are not live yet are added.  Either every item gets its room or nothing
        changes and ``OutOfPages`` is raised.  Returns each item's start position."""
        seen = set()
        new = []
        for req, n in items:
            if req in seen:
                raise ValueError(f"request {req!r} appears twice in one step")
            seen.add(req)
            if n < 1:
                raise ValueError(f"request {req!r} brings no tokens")
            if req not in self._lengths:
                new.append(req)
        if len(new) > self.state_slots.num_free:
            raise OutOfPages(
                f"{len(new)} new requests, {self.state_slots.num_free} request slots are free")
        need = [0] * len(self.groups)
        per_item = []
        for req, n in items:
            end = self._lengths.get(req, 0) + n
            if max_position is not None and end > max_position:
                raise ValueError(
                    f"request {req!r} would reach {end} tokens; the model allows {max_position}")
            mine = self.pages_needed(req, n)
            per_item.append(mine)
            for g, k in enumerate(mine):
                need[g] += k
        for g, k in enumerate(need):
            if k > self.groups[g].pool.num_free:
                raise OutOfPages(
                    f"the step needs {k} pages of group {g}, {self.groups[g].pool.num_free} are free")
        for req in new:
            self.add_request(req)
        starts = []
        for (req, n), mine in zip(items, per_item):          # the pages are there: hand them out
            for k, g in zip(mine, self.groups):
                if k:
                    g.tables[req].extend(g.pool.take() for _ in range(k))
            starts.append(self._lengths[req])
            self._lengths[req] += n
        return starts

    def release_passed(self, req: Hashable) -> int:
        """Give back pages that lie wholly behind a window.  Returns how many were freed."""
        freed = 0
        length = self._lengths[req]
        for g in self.groups:
            if g.spec.window is None:
                continue
            table = g.tables[req]
            for b in range(min(g.first_needed_block(length), len(table))):
                if table[b] != RELEASED:
                    g.pool.give_back(table[b])
                    table[b] = RELEASED
                    freed += 1
        if freed:
            self._touch(req)
        return freed

    def free_request(self, req: Hashable) -> None:
        if req not in self._lengths:
            raise KeyError(f"request {req!r} is not live")
        for g in self.groups:
            for page in g.tables.pop(req):
                if page != RELEASED:
                    g.pool.give_back(page)
        self.state_slots.give_back(self._state_slot.pop(req))
        del self._lengths[req]
        del self._version[req]

    # ---- what a step reads ----------------------------------------------------------------
    def block_table(self, group: int, req: Hashable) -> list[int]:
        return self.groups[group].tables[req]

    def max_blocks(self, reqs: Sequence[Hashable]) -> int:
        return max((len(g.tables[r]) for g in self.groups for r in reqs), default=0)

    def group_of_slot(self, cache_slot: int) -> Optional[int]:
        ent = self._slot_group.get(cache_slot)
        return None if ent is None else ent[0]

    def view(self, cache_slot: int, writes: bool, block_tables: Sequence[torch.Tensor],
             state_slots: Optional[torch.Tensor]):
        """The view of ``cache_slot`` for one step, given this step's device tables."""
        if cache_slot in self._slot_group:
            g, idx = self._slot_group[cache_slot]
            grp = self.groups[g]
            pages = None if grp.storage is None else grp.storage[idx]
            return PagedKVView(pages, block_tables[g], self.page_size, writes)
        if cache_slot in self._state_specs:
            return StateView(self._state_storage.get(cache_slot), state_slots, writes)
        return None

    # ---- accounting ----------------------------------------------------------------------
    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or freed twice; tables and pools agree."""
        for g in self.groups:
            g.pool.check()
            held = [p for t in g.tables.values() for p in t if p != RELEASED]
            if len(held) != len(set(held)):
                raise AssertionError("a page appears in two block tables")
            if set(held) != g.pool._held:
                raise AssertionError("block tables and the pool disagree on held pages")
        self.state_slots.check()
        if sorted(self._state_slot.values()) != sorted(self.state_slots._held):
            raise AssertionError("state slots and live requests disagree")
