"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
import random

import pytest
import torch

from fakes import fake_blocks, llama_like_manager
from sharpinference_b200.cache import CacheError, CacheManager, FreeList, OutOfPages, OutOfSlots
from sharpinference_b200.models.model import ScheduleEntry
from sharpinference_b200.parts.base import CacheSpec, StateSpec


def test_free_list_refuses_double_free_and_strangers():
    f = FreeList(3)
    a, b = f.take(), f.take()
    assert (a, b) == (0, 1) and f.free_count == 1 and f.held_count == 2
    f.give_back(a)
    with pytest.raises(CacheError):
        f.give_back(a)
    with pytest.raises(CacheError):
        f.give_back(2)          # never taken
    with pytest.raises(CacheError):
        f.give_back(7)
    assert f.take() == 0        # a freed id is handed out again


def test_groups_follow_cache_specs():
    m = llama_like_manager(layers=6, nope=(2, 5))
    assert len(m.groups) == 2
    chunk, full = m.groups
    assert chunk.spec.kind == "chunk" and chunk.entries == [0, 1, 3, 4]
    assert full.spec.kind == "full" and full.entries == [2, 5]
    slots = m.layer_slots()
    assert [s.group for s in slots] == [0, 0, 1, 0, 0, 1]


def test_reserve_commit_free_and_reuse():
    m = llama_like_manager(num_pages=4, page_size=4, chunk=8)
    m.add_request("a")
    assert m.pages_needed("a", 5) == {0: 2, 1: 2}
    m.reserve([("a", 5)])
    assert m.free_pages() == {0: 2, 1: 2}
    m.commit("a", 5)
    assert m.pages_needed("a", 3) == {0: 0, 1: 0}           # room left in the second page
    assert m.pages_needed("a", 4) == {0: 1, 1: 1}
    m.check_invariants()
    held = list(m.get("a").tables[1])
    m.free_request("a")
    assert m.free_pages() == {0: 4, 1: 4}
    with pytest.raises(CacheError):
        m.free_request("a")
    m.add_request("b")
    m.reserve([("b", 16)])
    assert sorted(m.get("b").tables[1]) == [0, 1, 2, 3] and set(held) <= set(m.get("b").tables[1])
    m.check_invariants()


@pytest.mark.parametrize("pos", [7, 8, 9])
def test_chunk_pages_are_released_at_the_chunk_edge(pos):
    """Chunk of 8 positions, pages of 4: once the next position is in a later chunk, the pages of
    the earlier chunk go back; before that none does.  The full group keeps everything."""
    m = llama_like_manager(num_pages=8, page_size=4, chunk=8)
    m.add_request("a")
    m.reserve([("a", pos)])
    m.commit("a", pos)                       # next position to be written is `pos`
    chunk_table, full_table = m.get("a").tables[0], m.get("a").tables[1]
    if pos < 8:
        assert all(p >= 0 for p in chunk_table)
    else:
        assert chunk_table[0] == -1 and chunk_table[1] == -1 and all(p >= 0 for p in chunk_table[2:])
    assert all(p >= 0 for p in full_table)
    m.check_invariants()


def test_window_group_releases_behind_the_window():
    blocks = fake_blocks([CacheSpec("window", 6, 1, 8)])
    m = CacheManager([ScheduleEntry(0)], blocks, page_size=4, num_pages=5, max_requests=2, dtype=torch.float32,
                     device="cpu", allocate=False)
    m.add_request("a")
    total = 0
    for n in (3, 4, 2, 5, 6):
        m.reserve([("a", n)])
        m.commit("a", n)
        total += n
        lo = max(0, total - 6 + 1)
        table = m.get("a").tables[0]
        for b, page in enumerate(table):
            assert (page < 0) == ((b + 1) * 4 <= lo), (total, b, table)
        m.check_invariants()
    assert m.held_pages("a")[0] <= 3


def test_out_of_pages_takes_nothing():
    m = llama_like_manager(num_pages=3, page_size=4)
    m.add_request("a")
    m.add_request("b")
    m.reserve([("a", 8)])
    m.commit("a", 8)
    before = m.free_pages()
    with pytest.raises(OutOfPages) as exc:
        m.reserve([("a", 1), ("b", 5)])
    assert exc.value.needed == 3 and exc.value.free == 1
    assert m.free_pages() == before and m.get("b").tables == {0: [], 1: []}
    assert not m.can_reserve([("b", 5)]) and m.can_reserve([("b", 4)])
    m.check_invariants()


def test_state_slots_are_assigned_and_returned():
    m = llama_like_manager(max_requests=2)
    a, b = m.add_request("a"), m.add_request("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(OutOfSlots):
        m.add_request("c")
    with pytest.raises(CacheError):
        m.add_request("a")
    m.free_request("a")
    assert m.add_request("c").state_slot == a.state_slot
    m.check_invariants()


def test_state_tensors_are_zeroed_on_assignment():
    blocks = fake_blocks([CacheSpec("full", 0, 1, 8), None], [None, StateSpec((3,), torch.float32)])
    m = CacheManager([ScheduleEntry(0), ScheduleEntry(1)], blocks, page_size=4, num_pages=2, max_requests=2,
                     dtype=torch.float32, device="cpu")
    slots = m.layer_slots()
    assert slots[0].state is None and slots[1].state.shape == (2, 3) and slots[1].kv is None
    assert slots[0].kv.shape == (2, 2, 1, 4, 8)
    r = m.add_request("a")
    slots[1].state[r.state_slot] += 5.0
    m.free_request("a")
    r2 = m.add_request("b")
    assert r2.state_slot == r.state_slot and float(slots[1].state[r2.state_slot].abs().sum()) == 0.0


def test_borrowed_cache_shares_the_group_and_adds_no_layer():
    spec = CacheSpec("full", 0, 1, 8)
    blocks = fake_blocks([spec, spec])
    m = CacheManager([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_from=0), ScheduleEntry(0)], blocks,
                     page_size=4, num_pages=2, max_requests=1, dtype=torch.float32, device="cpu")
    assert m.groups[0].entries == [0, 1, 3] and m.groups[0].kv.shape[0] == 3
    slots = m.layer_slots()
    assert slots[2].kv.data_ptr() == slots[0].kv.data_ptr() and not slots[2].writes_cache
    assert slots[3].kv.data_ptr() != slots[0].kv.data_ptr() and slots[3].writes_cache


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = llama_like_manager(num_pages=10, page_size=4, chunk=8, max_requests=4, layers=5, nope=(1, 4))
    live, next_id = {}, 0
    for _ in range(300):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.4 and live:
            rid = rng.choice(list(live))
            m.free_request(rid)
            del live[rid]
        elif live:
            ids = rng.sample(list(live), rng.randint(1, len(live)))
            wants = [(rid, rng.choice([1, 1, 1, 2, 3, 7, 13])) for rid in ids]
            try:
                m.reserve(wants)
            except OutOfPages:
                m.check_invariants()
                victim = max(live, key=lambda r: m.held_pages(r)[1])
                m.free_request(victim)
                del live[victim]
                continue
            for rid, n in wants:
                m.commit(rid, n)
                live[rid] += n
                rc = m.get(rid)
                assert rc.length == live[rid]
                # every position a later query can read is backed by a page
                for g in m.groups:
                    lo = g.spec.lowest_visible(rc.length)
                    for pos in range(lo, rc.length):
                        assert rc.tables[g.index][pos // 4] >= 0
        m.check_invariants()
    for rid in list(live):
        m.free_request(rid)
    assert m.free_pages() == {0: 10, 1: 10} and m.state_slots.free_count == 4


def test_pages_per_group_follow_what_each_group_can_hold():
    """Sizing from a memory budget: a group that forgets the past gets what max_batch requests can hold of it
    (span + a step + a page each), the rest goes to the groups that keep everything."""
    from fakes import fake_blocks
    from sharpinference_b200.cache import group_layout, pages_per_group
    from sharpinference_b200.models.model import ScheduleEntry
    from sharpinference_b200.parts.base import CacheSpec
    chunk, full = CacheSpec("chunk", 8192, 8, 128), CacheSpec("full", 0, 8, 128)
    blocks = fake_blocks([chunk, chunk, chunk, full] * 2)
    groups = group_layout([ScheduleEntry(i) for i in range(8)], blocks)
    assert groups == [(chunk, 6), (full, 2)]
    per_token = 2 * 8 * 128 * 2
    pages = pages_per_group(groups, budget_bytes=12 << 30, itemsize=2, page_size=64, max_batch=8, max_tokens_per_step=2048)
    # the chunked group: 8 requests x (8192 + 2048 + 64) positions
    assert pages[0] == 8 * (8192 + 2048 + 64) // 64
    spent = pages[0] * 64 * per_token * 6
    assert pages[1] == (((12 << 30) - spent) // (per_token * 2)) // 64
    assert pages[1] * 64 > 4 * pages[0] * 64                     # far more history than one size for all would give
    # a budget too small for the bound: the forgetting group takes half, never nothing
    small = pages_per_group(groups, budget_bytes=1 << 30, itemsize=2, page_size=64, max_batch=8, max_tokens_per_step=2048)
    assert small[0] * 64 * per_token * 6 <= (1 << 29) and small[0] >= 1 and small[1] >= 1
    # only forgetting groups: their bound, whatever the budget allows beyond it
    alone = pages_per_group([(chunk, 4)], budget_bytes=100 << 30, itemsize=2, page_size=64, max_batch=2, max_tokens_per_step=128)
    assert alone == [2 * (8192 + 128 + 64) // 64]
    assert pages_per_group([], budget_bytes=1, itemsize=2, page_size=64, max_batch=1, max_tokens_per_step=1) == []
