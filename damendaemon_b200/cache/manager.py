"""The cache manager: paged keys/values per layer group, block tables, per-request state slots.

Layers declare what they need: a paged need (``PagedKeyValues``, or any other ``PagedNeed``
that says what a page of it looks like) and/or a ``RequestState``. Layers whose paged need
is the same (for keys and values: heads, head size, window) form a *group*: one page pool,
one block table per request, one arena ``[layers, pages, *page shape]`` (for keys and values
``[layers, pages, 2, kv_heads, page_size, head_dim]``) in which a page index means the same
page in every layer of the group. Groups with
different needs (all keys; a window of them) have pages of their own. Pages are given
back when a request ends or, in a window group, once the window has passed them, and
are handed out again (last freed, first reused).

A request also owns one *slot*, a row index below ``max_requests``; per-request state of
fixed size lives at ``state[layer][slot]`` and is zeroed when the slot is taken. GPT-2
has no such state; the slots are kept for mixers that do (the reference keeps
``[max_batch, ...]`` state tensors indexed by slot, damendaemon/hybrid.py:486-487).

The reference's paged executor reserves a whole request at admission and never preempts
(damendaemon/paged.py:46-56, damendaemon/scheduler.py:763-780); ``reserve`` does the same
through page promises, while ``extend`` lets a caller without a reservation (trace
replay) grow step by step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from .pages import PageCapacityError, PagePool


class PagedNeed:
    """Per-token storage that grows with the request, kept in pages. A mixer may define its own (a frozen dataclass
    that derives from this, so that equal needs compare equal and share a group): it gives ``window`` (None: every
    earlier token stays; n: the last n), the shape of one page and a short label. The manager needs no more."""
    window: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        raise NotImplementedError

    @property
    def label(self) -> str:
        raise NotImplementedError


@dataclass(frozen=True)
class PagedKeyValues(PagedNeed):
    kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every earlier key stays; n: the last n keys

    def page_shape(self, page_size):
        return (2, self.kv_heads, page_size, self.head_dim)      # key plane and value plane, head-major inside a page

    @property
    def label(self):
        return f"kv{self.kv_heads}x{self.head_dim}"


@dataclass(frozen=True)
class RequestState:
    shape: Tuple[int, ...]
    dtype: str = "float32"


class CacheGroup:
    def __init__(self, need: PagedNeed, layers, n_pages, page_size, max_requests, max_blocks):
        self.need, self.layers = need, list(layers)
        self.pool = PagePool(n_pages, page_size)
        self.page_shape = tuple(int(n) for n in need.page_shape(page_size))
        self.tables = {}        # request id -> list of page ids, -1 where a page was given back
        self.arena = None       # device tensor [len(layers), n_pages, *page_shape]
        # the same block tables by slot, ready to be copied to the device: -1 = no page
        self.table_array = np.full((max_requests, max_blocks), -1, dtype=np.int32)

    @property
    def name(self):
        w = "all" if self.need.window is None else f"w{self.need.window}"
        return f"{self.need.label}.{w}"

    def first_needed_block(self, length: int) -> int:
        """Blocks before this one hold only keys that no later query can see."""
        if self.need.window is None:
            return 0
        return max(0, length - self.need.window + 1) // self.pool.page_size

    def pages_to_reach(self, request, length: int) -> int:
        table = self.tables.get(request, [])
        return max(0, self.pool.pages_for(length) - len(table))

    def peak_pages(self, total_tokens: int, max_step_tokens: int) -> int:
        """Most pages a request of total_tokens can hold at once (for promises)."""
        full = self.pool.pages_for(total_tokens)
        if self.need.window is None:
            return full
        return min(full, self.pool.pages_for(self.need.window - 1 + max_step_tokens) + 1)


class CacheManager:
    def __init__(self, layer_needs, kv_tokens: int, page_size: int, max_requests: int, max_context: int):
        """layer_needs: one list of PagedKeyValues / RequestState needs per cache site (a stop of the
        model's run order; the "layers" of a group below are these indices)."""
        if type(page_size) is not int or page_size <= 0:
            raise ValueError("page size must be a positive integer")
        if type(kv_tokens) is not int or kv_tokens < page_size:
            raise ValueError("the cache needs room for at least one page")
        if type(max_requests) is not int or max_requests <= 0:
            raise ValueError("max_requests must be positive")
        self.page_size, self.max_requests, self.max_context = page_size, max_requests, max_context
        self.max_blocks = (max_context + page_size - 1) // page_size
        n_pages = kv_tokens // page_size
        by_need = {}
        self.state_needs = {}                     # layer -> RequestState
        for layer, needs in enumerate(layer_needs):
            for need in needs or ():
                if isinstance(need, PagedNeed):
                    by_need.setdefault(need, []).append(layer)
                elif isinstance(need, RequestState):
                    self.state_needs[layer] = need
                else:
                    raise TypeError(f"layer {layer}: unknown cache need {need!r}")
        self.groups = [CacheGroup(need, layers, n_pages, page_size, max_requests, self.max_blocks)
                       for need, layers in by_need.items()]
        self.group_of_layer = {layer: g for g in self.groups for layer in g.layers}
        self.state = {}                           # layer -> device tensor [max_requests, *shape]
        self._free_slots = list(reversed(range(max_requests)))
        self.slot_of = {}                         # request id -> slot
        self.length = {}                          # request id -> tokens in the cache

    # ---- device storage ----
    def bytes_needed(self, element_size):
        """Bytes that allocate() takes on the device: the page arenas (elements of element_size bytes) and the
        per-request state rows."""
        import math
        total = 0
        for g in self.groups:
            total += len(g.layers) * g.pool.n_pages * math.prod(g.page_shape) * element_size
        widths = {"float32": 4, "bfloat16": 2, "float16": 2, "int32": 4, "int64": 8, "float64": 8}
        for need in self.state_needs.values():
            total += self.max_requests * math.prod(need.shape) * widths.get(need.dtype, 4)
        return total

    def allocate(self, device, dtype):
        import torch
        for g in self.groups:
            g.arena = torch.zeros((len(g.layers), g.pool.n_pages, *g.page_shape), device=device, dtype=dtype)
        for layer, need in self.state_needs.items():
            self.state[layer] = torch.zeros((self.max_requests, *need.shape), device=device,
                                            dtype=getattr(torch, need.dtype))

    def layer_view(self, layer, writable=True):
        """What a mixer sees of the cache: its group's arena slice and its state rows.
        ``layer`` counts the entries of ``layer_needs`` (the stops of the model's run order)."""
        g = self.group_of_layer.get(layer)
        return LayerCache(group=g, kv=None if g is None or g.arena is None else g.arena[g.layers.index(layer)],
                          state=self.state.get(layer), page_size=self.page_size, writable=writable)

    def bytes_per_token(self, element_size):
        import math
        return sum(len(g.layers) * math.prod(g.page_shape) // self.page_size * element_size for g in self.groups)

    # ---- requests ----
    def admit(self, request) -> int:
        if request in self.slot_of:
            raise ValueError(f"request {request!r} is already live")
        if not self._free_slots:
            raise PageCapacityError("no free request slot")
        slot = self._free_slots.pop()
        self.slot_of[request], self.length[request] = slot, 0
        for g in self.groups:
            g.tables[request] = []
        for tensor in self.state.values():
            tensor[slot].zero_()
        return slot

    def reserve(self, request, total_tokens: int, max_step_tokens: int):
        """Promise the pages a request of total_tokens will need; raises PageCapacityError
        (the request can wait) or ValueError (it can never fit) without changing anything."""
        wants = []
        for g in self.groups:
            n = g.peak_pages(total_tokens, max_step_tokens)
            if n > g.pool.n_pages:
                raise ValueError(f"a request of {total_tokens} tokens needs {n} pages; the pool has {g.pool.n_pages}")
            wants.append(n)
        for g, n in zip(self.groups, wants):
            current = max(g.pool._promised.get(request, 0), g.pool.held(request))
            if max(0, n - current) > g.pool.unpromised_pages:
                raise PageCapacityError(f"group {g.name}: {n} pages wanted, {g.pool.unpromised_pages} without a claim")
        for g, n in zip(self.groups, wants):
            g.pool.promise(request, n)

    def can_extend(self, growth) -> bool:
        """growth: [(request, new_length)]; True if extend(growth) would succeed."""
        for g in self.groups:
            beyond = 0
            total = 0
            for request, new_length in growth:
                n = g.pages_to_reach(request, new_length)
                within = max(0, g.pool._promised.get(request, 0) - g.pool.held(request))
                beyond += max(0, n - within)
                total += n
            if beyond > g.pool.unpromised_pages or total > g.pool.free_pages:
                return False
        return True

    def extend(self, growth):
        """Give every request in growth the pages to hold new_length tokens, all or nothing."""
        seen = set()
        for request, new_length in growth:
            if request not in self.slot_of:
                raise ValueError(f"request {request!r} is not live")
            if request in seen:
                raise ValueError(f"request {request!r} appears twice")
            seen.add(request)
            if new_length > self.max_context:
                raise ValueError(f"request {request!r}: {new_length} tokens exceed the context of {self.max_context}")
            if new_length < self.length[request]:
                raise ValueError(f"request {request!r} cannot shrink")
        if not self.can_extend(growth):
            raise PageCapacityError("the cache pages do not suffice for this step")
        for g in self.groups:
            for request, new_length in growth:
                n = g.pages_to_reach(request, new_length)
                if n:
                    table = g.tables[request]
                    start = len(table)
                    table.extend(g.pool.take(request, n))
                    g.table_array[self.slot_of[request], start:len(table)] = table[start:]

    def advance(self, request, new_length: int):
        """The request now holds new_length tokens; window groups give back what fell behind."""
        self.length[request] = new_length
        for g in self.groups:
            first = g.first_needed_block(new_length)
            table = g.tables[request]
            gone = [p for p in table[:first] if p >= 0]
            if gone:
                g.pool.give_back(request, gone)
                for i in range(min(first, len(table))):
                    table[i] = -1
                g.table_array[self.slot_of[request], :min(first, len(table))] = -1

    def release(self, request):
        """Give back every page and the slot. Safe to call for a request that is not live."""
        if request not in self.slot_of:
            return
        for g in self.groups:
            table = g.tables.pop(request)
            g.pool.give_back(request, [p for p in table if p >= 0])
            g.pool.forget(request)
            g.table_array[self.slot_of[request]] = -1
        self._free_slots.append(self.slot_of.pop(request))
        del self.length[request]

    def block_row(self, group, request):
        return group.tables[request]

    def check(self):
        for g in self.groups:
            g.pool.check()
            owned = {}
            for request, table in g.tables.items():
                for p in table:
                    if p >= 0:
                        assert p not in owned, f"page {p} is in two block tables"
                        owned[p] = request
            assert len(owned) == g.pool.used_pages, "pages held outside any block table"
        assert len(set(self._free_slots)) == len(self._free_slots)
        assert len(self._free_slots) + len(self.slot_of) == self.max_requests

    @property
    def used_tokens(self):
        return max((g.pool.used_pages for g in self.groups), default=0) * self.page_size

    @property
    def high_water_tokens(self):
        return max((g.pool.high_water_pages for g in self.groups), default=0) * self.page_size


@dataclass
class LayerCache:
    group: Optional[CacheGroup]
    kv: object                 # this layer's pages [n_pages, *page shape] (keys and values: [n_pages, 2, kv_heads, page, head_dim])
    state: object
    page_size: int
    writable: bool = True      # False: this mixer reads another stop's cache and must not write it

    @property
    def pages(self):
        return self.kv
