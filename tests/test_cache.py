"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from burn_lm_b200.cache import Cache, CacheError, CacheFull, ContextLengthExceeded, IdAllocator
from burn_lm_b200.parts.base import CacheNeed
from burn_lm_b200.plan import ScheduleEntry


def test_id_allocator_invariants():
    a = IdAllocator(4, "thing")
    got = [a.acquire() for _ in range(4)]
    assert got == [0, 1, 2, 3] and a.free_count == 0
    with pytest.raises(CacheFull):
        a.acquire()
    a.release(2)
    with pytest.raises(CacheError, match="not held"):
        a.release(2)                       # freed twice
    with pytest.raises(CacheError, match="out of range"):
        a.release(9)
    assert a.acquire() == 2                # used again
    a.release(3); a.release(1)
    assert a.acquire() == 1                # lowest first
    with pytest.raises(CacheFull):
        a.acquire_many(5)


def make_cache(max_tokens=64 * 6, max_seqs=3, max_seq_len=64 * 4, runs=3, shared=False):
    kv = CacheNeed("kv", n_kv_heads=2, head_dim=16)
    state = CacheNeed("state", state_shape=(4,), state_dtype="float32")
    needs = [kv, state, kv][:runs]
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)][:runs]
    if shared:
        needs = [kv, None, state]
        schedule = [ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(2)]
    return Cache(needs, schedule, max_tokens, max_seqs, max_seq_len, torch.float32, torch.device("cpu"))


def test_groups_and_views():
    c = make_cache()
    assert c.n_pages == 6 and c.max_pages_per_seq == 4
    v0, v1, v2 = c.view(0), c.view(1), c.view(2)
    assert v0.kind == "kv" and v2.kind == "kv" and v1.kind == "state"
    assert tuple(v0.pool.shape) == (6, 2, 2, 64, 16) and v0.pool.data_ptr() != v2.pool.data_ptr()
    assert v0.block_table is v2.block_table                     # one group, one table
    assert tuple(v1.state.shape) == (3, 4)
    s = make_cache(shared=True)
    assert s.view(1).pool.data_ptr() == s.view(0).pool.data_ptr() and not s.view(1).writes and s.view(0).writes


def test_windowed_runs_get_storage_of_their_own():
    full = CacheNeed("kv", n_kv_heads=2, head_dim=16)
    win = CacheNeed("kv", n_kv_heads=2, head_dim=16, window=32)
    c = Cache([full, win, full, win], [ScheduleEntry(i) for i in range(4)], 256, 2, 256, torch.float32, torch.device("cpu"))
    assert c.view(0).block_table is c.view(2).block_table and c.view(1).block_table is c.view(3).block_table
    assert c.view(0).block_table is not c.view(1).block_table and c.view(1).window == 32


def test_a_windowed_group_gives_back_what_lies_before_the_window():
    """Two groups, one with a window of 100 keys: as a sequence grows, the windowed group holds only the pages that
    a token still to come can see (about window / 64 + 2), the other one all of them; nothing is lost or held
    twice, and what a second sequence is given are the pages the first one gave back."""
    full = CacheNeed("kv", n_kv_heads=2, head_dim=16)
    win = CacheNeed("kv", n_kv_heads=2, head_dim=16, window=100)
    c = Cache([full, win], [ScheduleEntry(0), ScheduleEntry(1)], 64 * 12, 2, 64 * 10, torch.float32, torch.device("cpu"))
    gf, gw = c._kv_groups
    assert not gf.need.window and gw.need.window == 100
    a = c.acquire()
    length = 0
    for grow in (70, 30, 1, 1, 200, 64, 1, 150):
        c.reserve([(a, length + grow)])
        length += grow
        c.set_length(a, length)
        live = gw.live_pages(a)
        assert None not in live and len(set(live)) == len(live)
        assert len(gf.live_pages(a)) == -(-length // 64) == len(gw.pages_of[a])
        assert len(live) + gw.pages.free_count == c.n_pages
        # the step that made the sequence this long still saw its keys from (length - grow) - 99 on
        assert gw.dropped[a] == max(0, (length - grow) - 99) // 64
    assert length == 517 and gw.dropped[a] == 4 and len(gw.live_pages(a)) == 5
    assert c.view(1).block_table[a, :4].tolist() == [0, 0, 0, 0]
    held = set(gw.live_pages(a))
    b = c.acquire()
    c.reserve([(a, 518), (b, 64 * 3)])  # a's next dead pages go back first; b is given pages (lowest first)
    assert not (set(gw.live_pages(b)) & set(gw.live_pages(a))) and gw.dropped[a] == (517 - 99) // 64
    assert set(gw.live_pages(b)) & held                       # among them pages that a held a moment ago
    c.release(a)
    c.release(b)
    assert gw.pages.free_count == gf.pages.free_count == c.n_pages and gw.dropped == [0, 0]


def test_reserve_release_and_reuse():
    c = make_cache()
    a, b = c.acquire(), c.acquire()
    c.reserve([(a, 65), (b, 64)])
    assert c.free_pages == 3
    assert len(set(c.view(0).block_table[a, :2].tolist()) | set(c.view(0).block_table[b, :1].tolist())) == 3
    c.reserve([(a, 100)])                  # same pages still
    assert c.free_pages == 3
    with pytest.raises(CacheFull):
        c.reserve([(a, 64 * 4), (b, 64 * 3)])       # needs 4 more, 3 free; nothing changes
    assert c.free_pages == 3
    with pytest.raises(ContextLengthExceeded) as e:
        c.reserve([(a, 64 * 4 + 1)])
    assert e.value.actual == 257 and e.value.maximum == 256
    c.release(a)
    assert c.free_pages == 5 and c.seq_len[a] == 0
    with pytest.raises(CacheError):
        c.release(a)                       # freed twice
    with pytest.raises(CacheError):
        c.reserve([(a, 5)])                # not held
    a2 = c.acquire()
    assert a2 == a                         # the slot is used again
    c.release(a2); c.release(b)
    assert c.free_pages == 6 and c.slots.held_count == 0


def test_state_is_zeroed_when_a_slot_starts():
    c = make_cache()
    s = c.acquire()
    c.view(1).state[s] = 7.0
    c.release(s)
    assert c.acquire() == s and float(c.view(1).state[s].abs().sum()) == 0.0


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 20, max_seqs=5, max_seq_len=64 * 8)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and c.slots.free_count:
            live[c.acquire()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            new = live[s] + rng.randint(1, 100)
            try:
                c.reserve([(s, new)])
                live[s] = new
                c.set_length(s, new)
            except (CacheFull, ContextLengthExceeded):
                pass
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        g = c._kv_groups[0]
        held = [p for s in range(c.max_seqs) for p in g.pages_of[s]]
        assert len(held) == len(set(held))                                   # no page held twice
        assert len(held) + g.pages.free_count == c.n_pages                   # none lost
        assert all(len(g.pages_of[s]) == -(-live[s] // 64) for s in live)    # exactly what lengths need
        assert c.slots.held_count == len(live)
    c.release_all()
    assert c.free_pages == c.n_pages and c.slots.free_count == c.max_seqs


def test_random_traffic_of_whole_steps_keeps_the_block_tables_right():
    """Steps that grow several sequences at once (one transfer of new block-table entries a group), in a cache of
    two groups of which one looks back over a window and gives pages back: after every step each live sequence's row
    of each group's table lists exactly the pages the group holds for it, at their places; no page is held twice or
    lost in either group; a step that does not fit changes nothing."""
    rng = random.Random(1)
    full = CacheNeed("kv", n_kv_heads=1, head_dim=16)
    win = CacheNeed("kv", n_kv_heads=1, head_dim=16, window=90)
    c = Cache([full, win], [ScheduleEntry(0), ScheduleEntry(1)], 64 * 24, 6, 64 * 10, torch.float32, torch.device("cpu"))
    live = {}
    refused = 0
    for _ in range(1500):
        op = rng.random()
        if op < 0.2 and c.slots.free_count:
            live[c.acquire()] = 0
        elif op < 0.85 and live:
            some = rng.sample(sorted(live), rng.randint(1, len(live)))
            growth = [(s, live[s] + rng.choice([1, 1, 1, rng.randint(2, 150)])) for s in some]
            free_before = [g.pages.free_count for g in c._kv_groups]
            try:
                c.reserve(growth)
                for s, n in growth:
                    live[s] = n
                    c.set_length(s, n)
            except (CacheFull, ContextLengthExceeded):
                refused += 1
                # (the windowed group may have given pages back before the step was refused; nothing was acquired)
                assert all(g.pages.free_count >= f for g, f in zip(c._kv_groups, free_before))
        elif live:
            s = rng.choice(sorted(live))
            c.release(s)
            del live[s]
        for g in c._kv_groups:
            held = [p for s in range(c.max_seqs) for p in g.live_pages(s)]
            assert len(held) == len(set(held)) and len(held) + g.pages.free_count == c.n_pages
            for s, n in live.items():
                assert len(g.pages_of[s]) == -(-n // 64)
                row = g.block_table[s].tolist()
                for i, p in enumerate(g.pages_of[s]):
                    assert (p is None and i < g.dropped[s]) or row[i] == p
                if g.need.window and n > 0:
                    assert g.dropped[s] <= max(0, n - g.need.window + 1) // 64      # nothing a coming token still sees
    assert refused > 0
    c.release_all()
    assert all(g.pages.free_count == c.n_pages for g in c._kv_groups)
