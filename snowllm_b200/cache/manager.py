"""The cache manager: pages with a block table per request, in groups, and state slots.

A *group* is a set of layers with the same need: ("paged", None) keeps every key,
("paged", W) keeps a window of W positions.  Each group has pages of its own (its own pool of
page ids and, per layer of the group, its own device tensor [pages, 2, kv heads, page_size,
head_dim]) and each request has one block table per group: entry i is the page that holds
positions [i*page_size, (i+1)*page_size), or -1 once a window has passed it and the page was
given back.  Beside the pages, every request holds one slot: layers with state of fixed size
keep a tensor [slots + 1, *shape] each, indexed by that slot.

What is given back when: a window group's pages as soon as no later query can reach them (at the
end of the step that passed them); everything at ``free``.  The step function never allocates:
``ensure`` must have succeeded for the tokens it is given.
(the roles of snowllm/engine/block_manager.py, snowllm/engine/cache_resources.py:33-177 and
snowllm/context.py:15-40)"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import CapacityError
from ..parts.spec import PagedKVSpec, SlotStateSpec
from .pages import PagePool, StateSlots


@dataclass
class RequestCache:
    """What one live request holds."""
    slot: int
    tables: dict = field(default_factory=dict)        # group key -> list of page ids (-1: given back)
    num_tokens: int = 0                               # positions [0, num_tokens) are in the cache
    freed: bool = False
    synced: dict = field(default_factory=dict)        # group key -> table entries a host mirror already holds


@dataclass
class PagedView:
    pool: torch.Tensor
    block_table: torch.Tensor
    page_size: int


@dataclass
class SlotView:
    tensors: list


def pages_for(tokens: int, page_size: int) -> int:
    return -(-tokens // page_size)


class CacheManager:
    def __init__(self, cache_specs, page_size: int, num_pages, max_seqs: int,
                 dtype: torch.dtype = torch.float32, device=None):
        """``cache_specs``: {entry index -> PagedKVSpec | SlotStateSpec} for the run entries that own
        a cache.  ``num_pages``: an int for every group, or {group key -> int}.  ``device`` None
        keeps the book-keeping only (no tensors): what the CPU tests and sizing code use."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.max_seqs, self.dtype, self.device = page_size, max_seqs, dtype, device
        self.specs = dict(cache_specs)
        self.groups: dict[tuple, PagePool] = {}
        self.group_of: dict[int, tuple] = {}
        for idx, spec in self.specs.items():
            if isinstance(spec, PagedKVSpec):
                key = ("paged", spec.window)
                self.group_of[idx] = key
                if key not in self.groups:
                    n = num_pages[key] if isinstance(num_pages, dict) else num_pages
                    self.groups[key] = PagePool(int(n))
            elif not isinstance(spec, SlotStateSpec):
                raise TypeError(f"run entry {idx}: unknown cache spec {spec!r}")
        self.slots = StateSlots(max_seqs)
        self.pools: dict[int, torch.Tensor] = {}
        self.states: dict[int, list] = {}
        if device is not None:
            self._allocate()

    # -- device tensors -------------------------------------------------------------------
    def _allocate(self) -> None:
        for idx, spec in self.specs.items():
            if isinstance(spec, PagedKVSpec):
                n = self.groups[self.group_of[idx]].total
                self.pools[idx] = torch.zeros(max(n, 1), 2, spec.num_kv_heads, self.page_size, spec.head_dim,
                                              dtype=self.dtype, device=self.device)
            else:
                kinds = spec.dtypes or ("compute",) * len(spec.shapes)
                self.states[idx] = [
                    torch.zeros(self.max_seqs + 1, *shape, device=self.device,
                                dtype=self.dtype if kind == "compute" else torch.float32)
                    for shape, kind in zip(spec.shapes, kinds)]

    @staticmethod
    def bytes_per_page(cache_specs, page_size: int, dtype: torch.dtype) -> dict:
        """{group key -> bytes one page id costs over all layers of the group}."""
        esz = torch.empty((), dtype=dtype).element_size()
        out: dict[tuple, int] = {}
        for spec in cache_specs.values():
            if isinstance(spec, PagedKVSpec):
                key = ("paged", spec.window)
                out[key] = out.get(key, 0) + 2 * spec.num_kv_heads * page_size * spec.head_dim * esz
        return out

    # -- requests -------------------------------------------------------------------------
    def admit(self) -> RequestCache | None:
        """A slot and empty block tables, or None when every slot is taken."""
        slot = self.slots.alloc()
        if slot is None:
            return None
        return RequestCache(slot=slot, tables={key: [] for key in self.groups})

    def _first_needed_page(self, key, from_token: int) -> int:
        """First table entry that a query at position >= from_token can still reach."""
        window = key[1]
        if window is None:
            return 0
        return max(0, from_token - window + 1) // self.page_size

    def missing_pages(self, rc: RequestCache, total_tokens: int) -> dict:
        """{group key -> pages still to take} so that positions [num_tokens, total_tokens) fit."""
        need = {}
        want = pages_for(total_tokens, self.page_size)
        for key in self.groups:
            table = rc.tables[key]
            have = len(table)
            if key[1] is None:                         # every key is kept: the table has no holes
                need[key] = max(0, want - have)
                continue
            first = self._first_needed_page(key, rc.num_tokens)
            # entries below `first` are never needed again; entries [have, want) are new
            need[key] = max(0, want - max(have, first)) + sum(
                1 for i in range(first, min(have, want)) if table[i] < 0)
        return need

    def can_ensure(self, rc: RequestCache, total_tokens: int) -> bool:
        return all(n <= self.groups[k].free_count for k, n in self.missing_pages(rc, total_tokens).items())

    def ensure(self, rc: RequestCache, total_tokens: int) -> bool:
        """Take the pages that positions up to total_tokens need, in every group, or take nothing
        and return False."""
        if rc.freed:
            raise CapacityError("request was already freed")
        if not self.can_ensure(rc, total_tokens):
            return False
        want = pages_for(total_tokens, self.page_size)
        for key, pool in self.groups.items():
            table = rc.tables[key]
            if key[1] is not None:
                first = self._first_needed_page(key, rc.num_tokens)
                while len(table) < min(first, want):
                    table.append(-1)                   # positions a window has passed already
                for i in range(first, min(len(table), want)):
                    if table[i] < 0:
                        table[i] = pool.alloc(1)[0]
                        rc.synced[key] = min(rc.synced.get(key, 0), i)
            if want > len(table):
                table.extend(pool.alloc(want - len(table)))
        return True

    def commit(self, rc: RequestCache, total_tokens: int) -> None:
        """The step wrote positions up to total_tokens: record it, and give back the pages that a
        window has passed."""
        if total_tokens < rc.num_tokens:
            raise CapacityError("a request's cache cannot shrink")
        rc.num_tokens = total_tokens
        for key, pool in self.groups.items():
            if key[1] is None:
                continue
            table = rc.tables[key]
            for i in range(min(self._first_needed_page(key, total_tokens), len(table))):
                if table[i] >= 0:
                    pool.release([table[i]])
                    table[i] = -1
                    rc.synced[key] = min(rc.synced.get(key, 0), i)

    def free(self, rc: RequestCache) -> None:
        """Give back everything the request holds."""
        if rc.freed:
            raise CapacityError("request is freed twice")
        for key, pool in self.groups.items():
            pool.release([p for p in rc.tables[key] if p >= 0])
            rc.tables[key] = []
        self.slots.release(rc.slot)
        rc.freed = True
        rc.num_tokens = 0

    # -- facts ----------------------------------------------------------------------------
    def free_pages(self) -> dict:
        return {k: p.free_count for k, p in self.groups.items()}

    def min_free_pages(self) -> int:
        return min((p.free_count for p in self.groups.values()), default=1 << 30)

    def view(self, idx: int, block_tables: dict):
        """What the mixer of run entry ``idx`` gets: its pool and the step's block table of its
        group, or its state tensors."""
        if idx in self.pools:
            return PagedView(self.pools[idx], block_tables[self.group_of[idx]], self.page_size)
        if idx in self.states:
            return SlotView(self.states[idx])
        return None
