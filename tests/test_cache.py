"""The cache manager on the host: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; slots stay put."""

import random

import pytest
import torch

from gllm_b200.cache import BlockAllocator, CacheError, CacheManager, OutOfPages, SlotAllocator
from gllm_b200.parts.base import KVPageRequirement, StateRequirement


def manager(num_blocks=12, block_size=4, max_batch=3, window=None, two_groups=False, max_seq_len=None):
    reqs = [(KVPageRequirement.keys_and_values(2, 16, None), None, None), (KVPageRequirement.keys_and_values(2, 16, None), None, None)]
    if window is not None:
        reqs.append((KVPageRequirement.keys_and_values(2, 16, window), None, None))
    if two_groups:
        reqs.append((KVPageRequirement.keys_and_values(1, 32, None), None, None))
    return CacheManager(reqs, block_size, num_blocks, max_batch, max_seq_len or num_blocks * block_size,
                        torch.float32, "cpu", allocate_pools=False)


def test_allocator_rules():
    a = BlockAllocator(4)
    got = a.allocate(3)
    assert len(set(got)) == 3 and a.num_free == 1
    with pytest.raises(OutOfPages):
        a.allocate(2)
    assert a.num_free == 1                                  # nothing was taken
    a.free(got[:2])
    with pytest.raises(CacheError, match="nobody holds"):
        a.free([got[0]])                                    # freed twice
    with pytest.raises(CacheError, match="twice"):
        a.free([got[2], got[2]])
    with pytest.raises(CacheError, match="outside"):
        a.free([99])
    again = a.allocate(3)
    assert a.total_reused >= 2 and set(again) | {got[2]} == {0, 1, 2, 3}
    s = SlotAllocator(2)
    x, y = s.allocate(), s.allocate()
    assert {x, y} == {0, 1}
    with pytest.raises(OutOfPages):
        s.allocate()
    s.free(x)
    with pytest.raises(CacheError):
        s.free(x)


def test_layers_with_equal_needs_share_a_group():
    m = manager(window=6, two_groups=True)
    assert len(m.groups) == 3
    assert m.groups[0].owner_entries == [0, 1] and m.groups[1].window == 6
    caches = m.mixer_caches()
    assert [c.group for c in caches] == [0, 0, 1, 2]
    m2 = CacheManager([(KVPageRequirement.keys_and_values(2, 16), None, None), (KVPageRequirement.keys_and_values(2, 16), None, 0)],
                      4, 8, 2, 32, torch.float32, "cpu")
    c = m2.mixer_caches()
    assert c[1].group == 0 and not c[1].writes and c[0].writes
    assert c[1].pages.data_ptr() == c[0].pages.data_ptr()     # reads the other entry's pages
    assert m2.groups[0].pool.shape == (1, 8 + 1, 4 * 2 * 2 * 16)    # + the null page
    assert c[0].kv_pages().shape == (8 + 1, 2, 2, 4, 16)


def test_append_commit_free_and_slot_mapping():
    m = manager()
    rc = m.add_request("a")
    maps = m.append("a", 6)
    pages = m.requests["a"].blocks[0]
    assert len(pages) == 2
    assert list(maps[0]) == [pages[0] * 4 + i for i in range(4)] + [pages[1] * 4, pages[1] * 4 + 1]
    m.commit("a", 6)
    assert m.pages_needed("a", 2) == {0: 0} and m.pages_needed("a", 3) == {0: 1}
    maps = m.append("a", 3)
    assert list(maps[0][:2]) == [pages[1] * 4 + 2, pages[1] * 4 + 3]
    m.commit("a", 3)
    assert list(m.groups[0].block_table_host[rc.slot, :3]) == m.requests["a"].blocks[0]
    m.check_invariants()
    m.free_request("a")
    assert m.num_free_pages() == 12 and (m.groups[0].block_table_host[:-1] == -1).all()
    with pytest.raises(CacheError):
        m.free_request("a")


def test_out_of_pages_takes_nothing_and_rollback():
    m = manager(num_blocks=4, two_groups=True)
    m.add_request("a")
    m.append("a", 9)                                        # 3 pages in both groups
    m.commit("a", 9)
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.append("b", 5)                                    # needs 2, 1 free
    assert all(g.allocator.num_free == 1 for g in m.groups)
    assert not m.can_append("b", 5) and m.can_append("b", 4)
    m.append("b", 4)
    m.rollback("b", 0)
    assert all(g.allocator.num_free == 1 for g in m.groups)
    m.check_invariants()
    with pytest.raises(CacheError, match="max_seq_len"):
        m.append("a", 100)


def test_window_group_gives_pages_back_early():
    m = manager(num_blocks=8, block_size=4, window=6)
    m.add_request("a")
    full, win = m.groups[0], m.groups[1]
    for step_tokens in (5, 4, 1, 1, 1, 8):
        m.append("a", step_tokens)
        m.commit("a", step_tokens)
        n = m.requests["a"].num_tokens
        live = [i for i, b in enumerate(m.requests["a"].blocks[1]) if b >= 0]
        # the next token (position n) sees keys n-5 .. n; every block holding one of them is still there
        first_needed = max(0, n - 6 + 1) // 4
        assert live and live[0] == first_needed, (n, live)
        assert all(b >= 0 for b in m.requests["a"].blocks[0])
        m.check_invariants()
    assert win.allocator.num_free > full.allocator.num_free
    slot = m.requests["a"].slot
    assert win.block_table_host[slot, 0] == -1
    m.free_request("a")
    assert win.allocator.num_free == 8 and full.allocator.num_free == 8


def test_state_slots_are_zeroed_and_stay_put():
    reqs = [(None, StateRequirement((3,), torch.float32), None), (KVPageRequirement.keys_and_values(1, 16), None, None)]
    m = CacheManager(reqs, 4, 8, 2, 32, torch.float32, "cpu")
    caches = m.mixer_caches()
    assert caches[0].state.shape == (2 + 1, 3) and caches[0].pages is None and caches[1].state is None
    a = m.add_request("a")
    caches[0].state[a.slot] = 7
    b = m.add_request("b")
    assert a.slot != b.slot
    with pytest.raises(OutOfPages):
        m.add_request("c")
    m.free_request("a")
    c = m.add_request("c")
    assert c.slot == a.slot and float(caches[0].state[c.slot].abs().sum()) == 0   # reused slot starts at zero
    assert m.requests["b"].slot == b.slot


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_pool_whole(seed):
    rnd = random.Random(seed)
    m = manager(num_blocks=24, block_size=4, max_batch=4, window=10, two_groups=True)
    live, counter = {}, 0
    for _ in range(600):
        action = rnd.random()
        if action < 0.25 and len(live) < 4:
            rid = f"r{counter}"
            counter += 1
            m.add_request(rid)
            live[rid] = 0
        elif action < 0.85 and live:
            rid = rnd.choice(sorted(live))
            n = rnd.choice([1, 1, 1, 2, 3, 7, 12])
            if m.can_append(rid, n):
                maps = m.append(rid, n)
                for g, sm in maps.items():
                    assert len(sm) == n and len(set(sm.tolist())) == n
                m.commit(rid, n)
                live[rid] += n
                assert m.requests[rid].num_tokens == live[rid]
            else:
                before = [g.allocator.num_free for g in m.groups]
                with pytest.raises(CacheError):
                    m.append(rid, n)
                assert before == [g.allocator.num_free for g in m.groups]
        elif live:
            rid = rnd.choice(sorted(live))
            m.free_request(rid)
            del live[rid]
        m.check_invariants()
        # two live requests never share a slot of memory
        for g in m.groups:
            held = [b for rc in m.requests.values() for b in rc.blocks[g.index] if b >= 0]
            assert len(held) == len(set(held)) == g.allocator.num_held
    for rid in list(live):
        m.free_request(rid)
    assert all(g.allocator.num_free == 24 for g in m.groups) and m.slots.num_free == 4
    assert all(g.allocator.total_reused > 0 for g in m.groups)
