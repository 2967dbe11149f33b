"""The cache manager: pages with a block table per request, in groups, and state slots.

A *group* is a set of layers with the same need: ("paged", None) keeps every key,
("paged", W) keeps a window of W positions.  Each group has pages of its own (its own pool of
page ids and, per layer of the group, device tensors of its own in the layout its spec chooses:
[pages, 2, kv heads, page_size, head_dim] for keys and values of one width) and each request has
one block table per group: entry i is the page that holds
positions [i*page_size, (i+1)*page_size), or -1 once a window has passed it and the page was
given back.  Beside the pages, every request holds one slot: layers with state of fixed size
keep a tensor [slots + 1, *shape] each, indexed by that slot.  A mixer may ask for several of these
at once (pages and a state of fixed size): its ``cache_spec()`` is then a tuple, and so is its view.

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
    pool: torch.Tensor                 # the first (for keys and values of one width: the only) pool tensor
    block_table: torch.Tensor
    page_size: int
    pools: tuple = ()                  # every pool tensor of the spec, in the order of ``pool_shapes``


@dataclass
class SlotView:
    tensors: list


def pages_for(tokens: int, page_size: int) -> int:
    return -(-tokens // page_size)


_CACHE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _as_tuple(spec) -> tuple:
    return tuple(spec) if isinstance(spec, (tuple, list)) else (spec,)


class CacheManager:
    def __init__(self, cache_specs, page_size: int, num_pages, max_seqs: int,
                 dtype: torch.dtype = torch.float32, device=None):
        """``cache_specs``: {entry index -> PagedKVSpec | SlotStateSpec | a tuple of them} for the run
        entries that own a cache.  ``num_pages``: an int for every group, or {group key -> int}.
        ``device`` None keeps the book-keeping only (no tensors): what the CPU tests and sizing code use."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.max_seqs, self.dtype, self.device = page_size, max_seqs, dtype, device
        self.specs = dict(cache_specs)
        self.groups: dict[tuple, PagePool] = {}
        for idx, entry in self.specs.items():
            for spec in _as_tuple(entry):
                if isinstance(spec, PagedKVSpec):
                    key = ("paged", spec.window)
                    if key not in self.groups:
                        n = num_pages[key] if isinstance(num_pages, dict) else num_pages
                        self.groups[key] = PagePool(int(n))
                    if spec.cache_dtype is not None and spec.cache_dtype not in _CACHE_DTYPES:
                        raise TypeError(f"run entry {idx}: cache dtype {spec.cache_dtype!r} "
                                        f"(known: {', '.join(_CACHE_DTYPES)})")
                elif not isinstance(spec, SlotStateSpec):
                    raise TypeError(f"run entry {idx}: unknown cache spec {spec!r}")
        self.slots = StateSlots(max_seqs)
        self._tensors: dict[int, tuple] = {}       # entry index -> per spec of the entry: its tensors
        if device is not None:
            self._allocate()

    # -- device tensors -------------------------------------------------------------------
    def _allocate(self) -> None:
        for idx, entry in self.specs.items():
            made = []
            for spec in _as_tuple(entry):
                if isinstance(spec, PagedKVSpec):
                    n = max(self.groups[("paged", spec.window)].total, 1)
                    dtype = _CACHE_DTYPES[spec.cache_dtype] if spec.cache_dtype else self.dtype
                    made.append(tuple(torch.zeros(shape, dtype=dtype, device=self.device)
                                      for shape in spec.pool_shapes(n, self.page_size)))
                else:
                    kinds = spec.dtypes or ("compute",) * len(spec.shapes)
                    made.append(tuple(
                        torch.zeros(self.max_seqs + 1, *shape, device=self.device,
                                    dtype=self.dtype if kind == "compute" else torch.float32)
                        for shape, kind in zip(spec.shapes, kinds)))
            self._tensors[idx] = tuple(made)

    def _each(self, kind):
        for idx, entry in self.specs.items():
            for spec, tensors in zip(_as_tuple(entry), self._tensors.get(idx, ())):
                if isinstance(spec, kind):
                    yield idx, spec, tensors

    def paged_tensors(self) -> list:
        """Every pool tensor (first dimension: pages), over all run entries."""
        return [t for _, _, ts in self._each(PagedKVSpec) for t in ts]

    def state_tensors(self) -> list:
        """Every tensor of fixed-size state (first dimension: slots + 1), over all run entries."""
        return [t for _, _, ts in self._each(SlotStateSpec) for t in ts]

    def bytes_per_token(self) -> int:
        """Bytes one cached position costs over all paged layers (pools as allocated)."""
        return sum(t[0].numel() * t.element_size() for t in self.paged_tensors()) // self.page_size

    @staticmethod
    def bytes_per_page(cache_specs, page_size: int, dtype: torch.dtype) -> dict:
        """{group key -> bytes one page id costs over all layers of the group}."""
        out: dict[tuple, int] = {}
        for entry in cache_specs.values():
            for spec in _as_tuple(entry):
                if isinstance(spec, PagedKVSpec):
                    key = ("paged", spec.window)
                    esz = torch.empty((), dtype=_CACHE_DTYPES[spec.cache_dtype] if spec.cache_dtype
                                      else dtype).element_size()
                    out[key] = out.get(key, 0) + spec.elements_per_page(page_size) * esz
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

    def pages_for_life(self, total_tokens: int) -> dict:
        """{group key -> pages a request of ``total_tokens`` can hold at once}: what a pool must have for the
        request to run alone.  (A window group holds fewer while it decodes, but a request that is admitted
        again after a preemption takes pages for all it has so far.)"""
        return {key: pages_for(total_tokens, self.page_size) for key in self.groups}

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
        """What the mixer of run entry ``idx`` gets: for a PagedKVSpec its pools and the step's block
        table of its group, for a SlotStateSpec its state tensors; a tuple of these, in the spec's
        order, when the mixer's ``cache_spec()`` is a tuple; None when it asked for nothing."""
        entry = self.specs.get(idx)
        if entry is None or idx not in self._tensors:
            return None
        views = []
        for spec, tensors in zip(_as_tuple(entry), self._tensors[idx]):
            if isinstance(spec, PagedKVSpec):
                views.append(PagedView(tensors[0], block_tables[("paged", spec.window)], self.page_size, tensors))
            else:
                views.append(SlotView(list(tensors)))
        return tuple(views) if isinstance(entry, (tuple, list)) else views[0]
