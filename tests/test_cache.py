"""The cache's bookkeeping (CPU): slots and pages are never lost, held twice or freed twice."""
import random

import pytest
import torch

from pico_engine.cache import Cache, CacheFull, CacheNeeds, CacheStateError, FreeList, KVNeed, PAGE, pages_for


def test_free_list_takes_lowest_first_and_refuses_double_free():
    f = FreeList(4, "page")
    assert f.take(2) == [0, 1] and f.free_count == 2
    f.give([0])
    assert f.take(1) == [0]                       # given back, used again
    with pytest.raises(CacheStateError):
        f.give([3])                               # never taken
    f.give([1])
    with pytest.raises(CacheStateError):
        f.give([1])                               # freed twice
    with pytest.raises(CacheFull):
        f.take(5)
    f.check()


def needs(window=None, layers=3, state=0):
    full = CacheNeeds(kv=KVNeed(2, 16, None), state_elems=state)
    win = CacheNeeds(kv=KVNeed(2, 16, window))
    return [full] + [win] * (layers - 1)


def test_groups_have_storage_of_their_own():
    c = Cache(needs(window=32) + [None], max_tokens=512, max_seqs=4, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 2 and c.groups[0].entries == [0] and c.groups[1].entries == [1, 2]
    # 8 pages for the sequences and the idle page behind them
    assert c.groups[0].k.shape == (1, 9, 2, PAGE, 16) and c.groups[1].v.shape == (2, 9, 2, PAGE, 16)
    assert c.groups[0].k.data_ptr() != c.groups[1].k.data_ptr()
    k, v = c.pools(2)
    assert k.shape == (9, 2, PAGE, 16) and k.data_ptr() == c.groups[1].k[1].data_ptr()
    assert 3 not in c.group_of


def test_idle_rows_take_nothing_from_the_sequences():
    """The idle slot and page (what the padding rows of a fixed-size step use) lie behind the slots and pages
    of the sequences: they are never handed out, hold no length, and may stand in a page table many times."""
    c = Cache(needs(window=32, state=4), max_tokens=128, max_seqs=2, dtype=torch.float32, device="cpu")
    assert c.idle_slot == 2 and c.idle_page == 2 and c.state[0].shape == (3, 4)
    a, b = c.open(), c.open()
    assert {a, b} == {0, 1} and c.length(c.idle_slot) == 0
    c.reserve(a, 64); c.reserve(b, 64)
    with pytest.raises(CacheFull):
        c.reserve(a, 65)
    table = c.page_table(0, [a, c.idle_slot, c.idle_slot, b], 2)
    assert table.tolist() == [[0, -1], [2, -1], [2, -1], [1, -1]]
    assert c.page_table(1, [c.idle_slot]).tolist() == [[2]]
    snap = c.snapshot_state()
    c.state[0][a].fill_(7.0)
    c.restore_state(snap)
    assert float(c.state[0].abs().sum()) == 0.0
    c.close(a); c.close(b); c.check()


def test_each_sequence_has_its_own_length_and_pages():
    c = Cache(needs(), max_tokens=640, max_seqs=3, dtype=torch.float32, device="cpu", allocate=False)
    a, b = c.open(), c.open()
    c.reserve(a, 70); c.advance(a, 70)
    c.reserve(b, 5); c.advance(b, 5)
    assert (c.length(a), c.length(b)) == (70, 5) and c.held_tokens() == 128 + 64
    t = c.page_table(0, [a, b])
    assert t.shape == (2, 2) and t[0].tolist() == [0, 1] and t[1].tolist() == [2, -1]
    c.reserve(b, 1); c.advance(b, 1)              # same page
    assert c.page_table(0, [b], 4).tolist() == [[2, -1, -1, -1]]
    c.check()
    c.close(a)
    d = c.open()
    assert d == a                                  # the slot is used again
    c.reserve(d, 1)
    assert c.page_table(0, [d]).tolist() == [[0]]  # and so is its first page
    with pytest.raises(CacheStateError):
        c.close(7)
    c.close(b); c.close(d)
    with pytest.raises(CacheStateError):
        c.close(d)
    assert all(g.pages.free_count == g.pages.n for g in c.groups) and c.slots.free_count == 3
    c.check()


def test_full_cache_is_an_error_not_an_overwrite():
    c = Cache(needs(), max_tokens=128, max_seqs=2, dtype=torch.float32, device="cpu", allocate=False)
    a, b = c.open(), c.open()
    c.reserve(a, 64); c.advance(a, 64); c.reserve(b, 64); c.advance(b, 64)
    with pytest.raises(CacheFull):
        c.reserve(a, 1)
    with pytest.raises(CacheFull):
        c.open()
    c.check()


def test_window_group_gives_pages_back_as_the_window_moves():
    c = Cache(needs(window=32), max_tokens=1024, max_seqs=2, dtype=torch.float32, device="cpu", allocate=False)
    s = c.open()
    c.reserve(s, 200); c.advance(s, 200)           # a prompt needs all its pages during its step
    full, win = c.groups[0], c.groups[1]
    assert full.table[s] == [0, 1, 2, 3]
    # the next query stands at 200 and sees keys >= 169: pages 0 and 1 (keys < 128) are gone
    assert win.table[s] == [-1, -1, 2, 3] and win.pages.held_count == 2
    for _ in range(120):
        c.reserve(s, 1); c.advance(s, 1)
    assert sum(p >= 0 for p in win.table[s]) <= 2 and len(full.table[s]) == pages_for(320)
    assert c.page_table(1, [s]).shape == (1, 5)
    c.check(); c.close(s); c.check()
    assert win.pages.free_count == win.pages.n


def test_state_is_zero_when_a_slot_is_taken():
    c = Cache(needs(state=5), max_tokens=128, max_seqs=2, dtype=torch.float32, device="cpu")
    assert c.state_entries == [0] and c.state_of(0).shape == (3, 5) and c.state_of(1) is None     # two sequences and the idle row
    s = c.open()
    c.state_of(0)[s] += 3.0
    c.close(s)
    assert c.open() == s and float(c.state_of(0)[s].abs().sum()) == 0.0


def test_random_traffic_keeps_the_books():
    rnd = random.Random(0)
    c = Cache(needs(window=32), max_tokens=64 * 40, max_seqs=6, dtype=torch.float32, device="cpu", allocate=False)
    live = []
    for _ in range(600):
        r = rnd.random()
        if r < 0.25 and len(live) < 6:
            live.append(c.open())
        elif r < 0.4 and live:
            c.close(live.pop(rnd.randrange(len(live))))
        elif live:
            s = rnd.choice(live)
            n = rnd.choice([1, 1, 1, 17, 64, 100])
            try:
                c.reserve(s, n)
                c.advance(s, n)
            except CacheFull:
                c.close(s); live.remove(s)
        c.check()
    for s in live:
        c.close(s)
    c.check()
    assert c.slots.free_count == 6 and all(g.pages.free_count == g.pages.n for g in c.groups)


def test_values_and_state_may_be_shaped_otherwise():
    """Keys and values need not have the same heads and head size (a cache of one compressed row per position keeps
    no values at all), and a mixer may ask for its state in another dtype."""
    needs_ = [CacheNeeds(kv=KVNeed(2, 16, None, v_head_dim=24)), CacheNeeds(kv=KVNeed(1, 40, None, v_heads=0)),
              CacheNeeds(kv=KVNeed(2, 16, None, v_head_dim=24), state_elems=6, state_dtype="bfloat16"),
              CacheNeeds(state_elems=3, state_dtype="engine")]
    c = Cache(needs_, max_tokens=128, max_seqs=2, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 2 and c.groups[0].entries == [0, 2]
    k, v = c.pools(2)
    assert k.shape == (3, 2, PAGE, 16) and v.shape == (3, 2, PAGE, 24)
    k, v = c.pools(1)
    assert k.shape == (3, 1, PAGE, 40) and v.numel() == 0
    assert c.state_of(2).dtype == torch.bfloat16 and c.state_of(3).dtype == torch.float32 and c.state_of(3).shape == (3, 3)
    assert c.bytes() == 4 * (2 * 3 * PAGE * (2 * 16 + 2 * 24) + 3 * PAGE * 40) + 3 * 6 * 2 + 3 * 3 * 4
    with pytest.raises(ValueError, match="state_dtype"):
        Cache([CacheNeeds(state_elems=2, state_dtype="int8")], 64, 1, torch.float32, "cpu")
