"""The cache manager's book-keeping: no page lost, held twice or freed twice, under random orders
of requests; window groups give pages back as the window passes; slots."""
import random

import pytest

from snowllm_b200.cache import CacheManager, PagePool, StateSlots
from snowllm_b200.errors import CapacityError
from snowllm_b200.parts.spec import PagedKVSpec, SlotStateSpec

SPECS = {0: PagedKVSpec(2, 16), 1: SlotStateSpec(((2, 8),)), 2: PagedKVSpec(2, 16),
         3: PagedKVSpec(1, 32, window=20)}


def held_pages(cm, live):
    out = {}
    for key in cm.groups:
        pages = [p for rc in live for p in rc.tables[key] if p >= 0]
        out[key] = pages
    return out


def check_invariants(cm, live):
    for key, pool in cm.groups.items():
        pages = held_pages(cm, live)[key]
        assert len(pages) == len(set(pages)), f"a page of {key} is held twice"
        assert len(pages) + pool.free_count == pool.total, f"a page of {key} is lost"
        assert not set(pages) & set(pool._free), "a held page is on the free list"
    slots = [rc.slot for rc in live]
    assert len(slots) == len(set(slots)) and len(slots) + cm.slots.free_count == cm.max_seqs


def test_pool_refuses_double_free_and_foreign_pages():
    pool = PagePool(4)
    a = pool.alloc(3)
    assert pool.alloc(2) is None and pool.free_count == 1
    pool.release(a[:1])
    with pytest.raises(CapacityError, match="twice"):
        pool.release(a[:1])
    with pytest.raises(CapacityError, match="belong"):
        pool.release([7])
    assert pool.alloc(1) == a[:1]           # the page just given back is handed out next


def test_slots():
    s = StateSlots(2)
    a, b = s.alloc(), s.alloc()
    assert {a, b} == {0, 1} and s.alloc() is None and s.dummy == 2
    s.release(a)
    with pytest.raises(CapacityError):
        s.release(a)
    assert s.alloc() == a


def test_groups_and_full_attention_pages():
    cm = CacheManager(SPECS, page_size=16, num_pages=8, max_seqs=3)
    assert set(cm.groups) == {("paged", None), ("paged", 20)}
    rc = cm.admit()
    assert cm.ensure(rc, 33) and len(rc.tables[("paged", None)]) == 3
    cm.commit(rc, 33)
    assert cm.ensure(rc, 34) and len(rc.tables[("paged", None)]) == 3     # same page
    assert cm.ensure(rc, 49) and len(rc.tables[("paged", None)]) == 4
    assert not cm.ensure(rc, 16 * 8 + 1)                                   # all or nothing
    assert len(rc.tables[("paged", None)]) == 4
    cm.free(rc)
    assert cm.free_pages() == {("paged", None): 8, ("paged", 20): 8}
    with pytest.raises(CapacityError):
        cm.free(rc)


def test_window_group_gives_pages_back_and_reuses_them():
    cm = CacheManager({0: PagedKVSpec(1, 16, window=20)}, page_size=16, num_pages=3, max_seqs=1)
    rc = cm.admit()
    key = ("paged", 20)
    total = 0
    for _ in range(40):                      # 40 steps of 7 tokens through a 3-page pool
        assert cm.ensure(rc, total + 7)
        total += 7
        cm.commit(rc, total)
        table = rc.tables[key]
        first_needed = max(0, total - 20 + 1) // 16
        assert all(p < 0 for p in table[:first_needed]) and all(p >= 0 for p in table[first_needed:])
        assert cm.groups[key].held() == len(table) - first_needed <= 3
    cm.free(rc)
    assert cm.groups[key].free_count == 3


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_books(seed):
    rng = random.Random(seed)
    cm = CacheManager(SPECS, page_size=rng.choice((4, 16)), num_pages=rng.randint(6, 40),
                      max_seqs=rng.randint(1, 5))
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.25:
            rc = cm.admit()
            if rc is None:
                assert len(live) == cm.max_seqs
            else:
                live.append(rc)
        elif op < 0.8 and live:
            rc = rng.choice(live)
            n = rng.choice((1, 1, 1, 2, 5, 17, 40))
            before = held_pages(cm, live)
            if cm.ensure(rc, rc.num_tokens + n):
                cm.commit(rc, rc.num_tokens + n)
            else:
                assert held_pages(cm, live) == before, "a failed ensure took pages"
        elif live:
            rc = live.pop(rng.randrange(len(live)))
            cm.free(rc)
        check_invariants(cm, live)
    for rc in live:
        cm.free(rc)
    check_invariants(cm, [])
    assert all(p.free_count == p.total for p in cm.groups.values())


def test_bytes_per_page():
    import torch
    b = CacheManager.bytes_per_page(SPECS, 16, torch.bfloat16)
    assert b[("paged", None)] == 2 * (2 * 2 * 16 * 16 * 2) and b[("paged", 20)] == 2 * 1 * 16 * 32 * 2


def test_spec_chooses_the_pool_layout_and_a_mixer_may_hold_pages_and_state():
    """Keys and values of one width share a tensor; of two widths they are two tensors; a cache of keys only
    (a latent row per position) is one; the cache dtype may differ from the compute dtype; a tuple of specs
    gives a tuple of views in the same order."""
    import torch
    specs = {0: PagedKVSpec(2, 16),
             1: PagedKVSpec(2, 16, v_head_dim=8),
             2: PagedKVSpec(1, 40, v_head_dim=0, cache_dtype="float32"),
             3: (PagedKVSpec(3, 8, window=32), SlotStateSpec(((5,), (2, 3)), ("f32", "compute"))),
             4: SlotStateSpec(((4,),))}
    cm = CacheManager(specs, page_size=4, num_pages={("paged", None): 6, ("paged", 32): 9}, max_seqs=2,
                      dtype=torch.bfloat16, device="cpu")
    tables = {key: torch.zeros(1, 3, dtype=torch.int32) for key in cm.groups}
    v0 = cm.view(0, tables)
    assert v0.pool.shape == (6, 2, 2, 4, 16) and v0.pool.dtype == torch.bfloat16 and len(v0.pools) == 1
    v1 = cm.view(1, tables)
    assert [tuple(t.shape) for t in v1.pools] == [(6, 2, 4, 16), (6, 2, 4, 8)] and v1.pool is v1.pools[0]
    v2 = cm.view(2, tables)
    assert [tuple(t.shape) for t in v2.pools] == [(6, 1, 4, 40)] and v2.pool.dtype == torch.float32
    paged, state = cm.view(3, tables)
    assert paged.pool.shape == (9, 2, 3, 4, 8) and paged.block_table is tables[("paged", 32)]
    assert [tuple(t.shape) for t in state.tensors] == [(3, 5), (3, 2, 3)]
    assert state.tensors[0].dtype == torch.float32 and state.tensors[1].dtype == torch.bfloat16
    assert cm.view(4, tables).tensors[0].shape == (3, 4) and cm.view(7, tables) is None
    assert len(cm.paged_tensors()) == 5 and len(cm.state_tensors()) == 3
    per_page = CacheManager.bytes_per_page(specs, 4, torch.bfloat16)
    assert per_page[("paged", None)] == (2 * 2 * 4 * 16) * 2 + (2 * 4 * 16 + 2 * 4 * 8) * 2 + (1 * 4 * 40) * 4
    assert per_page[("paged", 32)] == 2 * 3 * 4 * 8 * 2
    assert cm.bytes_per_token() == (per_page[("paged", None)] + per_page[("paged", 32)]) // 4
    with pytest.raises(TypeError, match="cache dtype"):
        CacheManager({0: PagedKVSpec(1, 8, cache_dtype="int8")}, 4, 2, 1)
    with pytest.raises(TypeError, match="unknown cache spec"):
        CacheManager({0: (PagedKVSpec(1, 8), "state")}, 4, 2, 1)
