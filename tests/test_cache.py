"""Cache bookkeeping on the CPU: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch


def _cache(pe, max_tokens=64 * 12, max_slots=4, max_seq_len=512, window=None, with_state=False):
    CR = pe.parts.CacheRequest
    reqs = {0: CR("kv", kv_heads=2, head_dim=16), 1: CR("kv", kv_heads=2, head_dim=16),
            2: CR("kv", kv_heads=2, head_dim=16, window=window) if window else CR("kv", kv_heads=2, head_dim=16)}
    if with_state:
        reqs[3] = CR("state", state_shapes=(("acc", (3, 5), "float32"),))
    return pe.cache.PagedCache(reqs, max_tokens=max_tokens, max_slots=max_slots, max_seq_len=max_seq_len,
                               dtype=torch.float32, device="cpu")


def test_groups_have_storage_of_their_own(pe):
    c = _cache(pe, window=100, with_state=True)
    kinds = [(g.request.kind, g.request.window, g.entries) for g in c.groups]
    assert kinds == [("kv", None, [0, 1]), ("kv", 100, [2]), ("state", None, [3])]
    assert c.groups[0].storage.shape == (2, 2, 12, 2, 64, 16)
    assert c.groups[1].storage.shape == (1, 2, 12, 2, 64, 16)
    assert c.groups[0].storage.data_ptr() != c.groups[1].storage.data_ptr()
    assert c.view(1).index == 1 and c.view(2).index == 0 and c.view(2).window == 100
    assert c.view(3).state("acc").shape == (4, 3, 5)


def test_slots_are_reused_and_never_held_twice(pe):
    c = _cache(pe)
    a, b = c.alloc_slot(), c.alloc_slot()
    assert a != b
    c.free_slot(a)
    assert c.alloc_slot() == a  # the slot just given back is used again at once
    c.alloc_slot(), c.alloc_slot()
    with pytest.raises(pe.cache.CacheFull):
        c.alloc_slot()
    c.check()


def test_double_free_and_unknown_slot(pe):
    c = _cache(pe)
    s = c.alloc_slot()
    c.free_slot(s)
    with pytest.raises(pe.cache.CacheBookkeepingError):
        c.free_slot(s)
    with pytest.raises(pe.cache.CacheBookkeepingError):
        c.free_slot(3)
    pool = pe.cache.NumberPool(3)
    n = pool.take()
    pool.give_back(n)
    with pytest.raises(pe.cache.CacheBookkeepingError):
        pool.give_back(n)
    with pytest.raises(pe.cache.CacheBookkeepingError):
        pool.give_back(7)


def test_pages_follow_lengths(pe):
    c = _cache(pe)
    s = c.alloc_slot()
    c.reserve(s, 5); c.commit(s, 5)
    assert len(c.groups[0].pages_of_slot[s]) == 1 and c.free_pages() == 11
    c.reserve(s, 64); c.commit(s, 64)
    assert len(c.groups[0].pages_of_slot[s]) == 1
    c.reserve(s, 65); c.commit(s, 65)
    assert len(c.groups[0].pages_of_slot[s]) == 2
    table = c.groups[0].page_table[s, :2].tolist()
    assert table == c.groups[0].pages_of_slot[s]
    c.free_slot(s)
    assert c.free_pages() == 12
    c.check()


def test_full_cache_raises_and_changes_nothing(pe):
    c = _cache(pe, max_tokens=64 * 3)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve(a, 128); c.commit(a, 128)
    before = (c.free_pages(), list(c.groups[0].pages_of_slot[b]))
    with pytest.raises(pe.cache.CacheFull):
        c.reserve(b, 129)
    assert (c.free_pages(), list(c.groups[0].pages_of_slot[b])) == before
    with pytest.raises(pe.cache.CacheFull):
        c.reserve(a, 513)  # beyond the longest sequence
    c.check()


def test_window_group_gives_pages_back(pe):
    c = _cache(pe, window=70, max_tokens=64 * 12)
    s = c.alloc_slot()
    c.reserve(s, 300); c.commit(s, 300)
    full, win = c.groups[0], c.groups[1]
    assert all(p >= 0 for p in full.pages_of_slot[s]) and len(full.pages_of_slot[s]) == 5
    # the next query sits at 300 and sees keys 231..300: pages 0..2 (positions < 192) are gone
    assert [p >= 0 for p in win.pages_of_slot[s]] == [False, False, False, True, True]
    assert win.pool.held_count == 2 and full.pool.held_count == 5
    c.check()
    c.free_slot(s)
    assert win.pool.held_count == 0 and full.pool.held_count == 0
    c.check()


def test_state_is_zero_for_a_new_sequence(pe):
    c = _cache(pe, with_state=True)
    s = c.alloc_slot()
    c.view(3).state("acc")[s] += 4.0
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and float(c.view(3).state("acc")[s2].abs().sum()) == 0.0


def test_truncate(pe):
    c = _cache(pe)
    s = c.alloc_slot()
    c.reserve(s, 200); c.commit(s, 200)
    c.truncate(s, 70)
    assert c.length(s) == 70 and len(c.groups[0].pages_of_slot[s]) == 2
    c.check()
    cw = _cache(pe, window=70)
    s = cw.alloc_slot()
    cw.reserve(s, 10); cw.commit(s, 10)
    with pytest.raises(pe.cache.CacheBookkeepingError):
        cw.truncate(s, 5)


def test_random_traffic_keeps_the_books(pe):
    rng = random.Random(0)
    c = _cache(pe, max_tokens=64 * 40, max_slots=6, max_seq_len=700, window=90)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.3 and len(live) < 6:
            live[c.alloc_slot()] = 0
        elif op < 0.5 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            new = min(700, live[s] + rng.choice([1, 1, 1, 17, 64, 130]))
            try:
                c.reserve(s, new)
            except pe.cache.CacheFull:
                continue
            c.commit(s, new)
            live[s] = new
        c.check()
        assert sorted(live) == c.live_slots
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pool.held_count == 0 for g in c.groups if g.pool)


def test_a_step_that_cannot_get_all_its_pages_takes_none(pe):
    """The runner reserves for every sequence of a step or for none (no device needed: only the books)."""
    runner_mod = __import__("importlib").import_module("pytorch-engine_b200.engine.runner")
    c = _cache(pe, max_tokens=64 * 6, window=100)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve(a, 64); c.commit(a, 64)
    c.reserve(b, 64); c.commit(b, 64)
    free = c.free_pages()

    class Books:
        cache = c
    with pytest.raises(pe.cache.CacheFull):
        runner_mod.ModelRunner._reserve_all(Books, [(a, 64 * 3), (b, 64 * 5)])   # the second cannot be met
    assert c.free_pages() == free and c.length(a) == 64
    c.check()
    runner_mod.ModelRunner._reserve_all(Books, [(a, 64 * 3), (b, 64 * 3)])
    assert c.free_pages() == free - 4
    c.release_reserved(a)
    assert c.free_pages() == free - 2
    c.check()


def test_decode_attention_ranges(pe):
    """How many ranges a sequence's keys are shared out over (the decision only; no device)."""
    f = pe.kernels.ops.decode_ranges
    assert f(296, 8 * 8, 4096, 512) == (0, 4, 512)   # batch 8, 8 kv heads: four ranges make one wave of 256 blocks
    assert f(296, 1 * 8, 4096, 512) == (0, 8, 512)   # batch 1: no more ranges than 512 keys each
    assert f(296, 1 * 8, 16384, 512) == (0, 32, 512)
    assert f(296, 1 * 8, 40960, 512) == (0, 37, 512)  # a roomy cache: 37 ranges in the grid, of at least 512 keys each
    assert f(296, 16 * 8, 4096, 512) == (0, 2, 512)
    assert f(296, 64 * 8, 4096, 512) == (0, 2, 2048)  # several waves anyway: ranges of about 2,048 keys
    assert f(296, 64 * 8, 32768, 512) == (0, 16, 2048)
    assert f(296, 64 * 8, 100, 512) == (0, 1, 2048)
    assert f(296, 3, 40, 512) == (0, 1, 512)          # a short context is one range
    for slots, pairs, kv in [(296, 7, 5000), (592, 100, 70000), (10, 1000, 64)]:
        sk, n, least = f(slots, pairs, kv, 512)
        assert sk == 0 and 1 <= n <= max(1, -(-kv // 512)) and least in (512, 2048)


def test_reset_forgets_everything_and_loses_nothing(pe):
    c = _cache(pe, window=100, with_state=True)
    slots = [c.alloc_slot() for _ in range(3)]
    for s, n in zip(slots, (200, 1, 130)):
        c.reserve(s, n)
        c.commit(s, n)
    c.view(3).state("acc")[slots[1]].fill_(7.0)
    assert c.free_pages() < 12
    c.reset()
    assert c.live_slots == [] and c.free_pages() == 12
    c.check()
    again = [c.alloc_slot() for _ in range(4)]            # every slot can be taken again, with its state at zero
    assert sorted(again) == [0, 1, 2, 3] and float(c.view(3).state("acc").abs().sum()) == 0.0
    c.reserve(again[0], 512)
    c.commit(again[0], 512)
    c.reset()
    c.reset()                                             # nothing live: nothing to do
    c.check()


def test_entries_of_a_block_with_two_mixers(pe):
    """A block with several mixers has one cache entry per mixer, keyed (entry, mixer name)."""
    CR = pe.parts.CacheRequest
    reqs = {0: CR("kv", kv_heads=2, head_dim=16), (1, "local"): CR("kv", kv_heads=2, head_dim=16, window=64),
            (1, "global"): CR("kv", kv_heads=2, head_dim=16), (1, "memory"): CR("state", state_shapes=(("m", (4,), "float32"),))}
    c = pe.cache.PagedCache(reqs, max_tokens=256, max_slots=2, max_seq_len=256, dtype=torch.float32, device="cpu")
    assert [(g.request.kind, g.request.window, g.entries) for g in c.groups] == [
        ("kv", None, [0, (1, "global")]), ("kv", 64, [(1, "local")]), ("state", None, [(1, "memory")])]
    assert c.view((1, "global")).index == 1 and c.view((1, "local")).window == 64
    assert c.view((1, "memory")).state("m").shape == (2, 4) and c.view((1, "nothing")) is None
