"""The cache's bookkeeping: slots and pages are never lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from tau_rs_b200.cache import PAGE_TOKENS, CacheFull, FreeList, SequenceCache, pages_for
from tau_rs_b200.parts import CacheNeed


def make(max_tokens=64 * 8, limit=64 * 5, slots=None, with_state=True):
    groups = {"attention": (CacheNeed("kv", n_kv_heads=2, head_dim=16), 3)}
    if with_state:
        groups["recurrent"] = (CacheNeed("state", state_shape=(4, 2), state_dtype=torch.float32), 2)
    return SequenceCache(groups, max_tokens, limit, torch.float32, torch.device("cpu"), slots)


def test_free_list_refuses_misuse():
    pool = FreeList(3, "page")
    taken = pool.take(2)
    assert taken == [0, 1] and pool.available == 1
    with pytest.raises(CacheFull):
        pool.take(2)
    pool.give_back([0])
    with pytest.raises(ValueError):
        pool.give_back([0])          # freed twice
    with pytest.raises(ValueError):
        pool.give_back([2])          # never taken
    with pytest.raises(ValueError):
        pool.give_back([7])
    assert pool.take(1) == [0]       # what came back goes out again first
    pool.check()


def test_shapes_and_sizing():
    cache = make(max_tokens=64 * 8 - 1)
    assert cache.n_pages == 8 and cache.pages_per_sequence == 5 and cache.max_sequence_tokens == 320
    view = cache.layer_view("attention", 2)
    assert view.keys.shape == (8, 2, PAGE_TOKENS, 16) and view.values.shape == view.keys.shape and view.group == "attention"
    assert cache.layer_view("recurrent", 1).state.shape == (8, 4, 2)
    assert cache.bytes_per_token() == 2 * 3 * 2 * 16 * 4 and pages_for(65) == 2 and pages_for(64) == 1


def test_sequences_take_pages_as_they_grow_and_give_them_back():
    cache = make()
    a, b = cache.open(), cache.open()
    cache.reserve(a, 65)
    cache.advance(a, 65)
    cache.reserve(b, 1)
    cache.advance(b, 1)
    assert cache.free_tokens() == 5 * 64 and cache.length(a) == 65
    rows = cache.page_rows("attention", [a, b], 2)
    assert rows.shape == (2, 2) and len({rows[0, 0], rows[0, 1], rows[1, 0]}) == 3
    cache.reserve(a, 100)            # still two pages
    assert cache.free_tokens() == 5 * 64
    with pytest.raises(CacheFull):
        cache.reserve(a, 321)        # beyond the longest sequence allowed
    with pytest.raises(CacheFull):
        cache.reserve(b, 64 * 6 + 1) # beyond what is free
    cache.check()
    cache.close(a)
    with pytest.raises(ValueError):
        cache.close(a)
    with pytest.raises(ValueError):
        cache.length(a)
    assert cache.free_tokens() == 7 * 64
    c = cache.open()
    assert c == a                    # the slot is used again
    assert cache.length(c) == 0
    cache.close(b)
    cache.close(c)
    cache.check()
    assert cache.free_tokens() == 8 * 64 and cache.slots.in_use == 0


def test_state_is_zero_for_a_new_sequence_only():
    cache = make()
    a = cache.open()
    state = cache.layer_view("recurrent", 0).state
    state[a] += 3.0
    b = cache.open()
    assert float(state[a].sum()) == 24.0 and float(state[b].sum()) == 0.0
    cache.close(a)
    assert cache.open() == a and float(state[a].sum()) == 0.0


def test_random_traffic_keeps_every_invariant():
    rng = random.Random(0)
    cache = make(max_tokens=64 * 12, limit=64 * 6, slots=5)
    live = {}
    for _ in range(2000):
        action = rng.random()
        if action < 0.3 and cache.slots.available:
            live[cache.open()] = 0
        elif action < 0.8 and live:
            slot = rng.choice(list(live))
            target = live[slot] + rng.randint(1, 90)
            try:
                cache.reserve(slot, target)
                cache.advance(slot, target)
                live[slot] = target
            except CacheFull:
                pass
        elif live:
            slot = rng.choice(list(live))
            cache.close(slot)
            del live[slot]
        cache.check()
        held = sum(pages_for(length) for length in live.values())
        assert cache.kv["attention"].pool.in_use >= held
    for slot in list(live):
        cache.close(slot)
    cache.check()
    assert cache.free_tokens() == 64 * 12


def test_a_window_gives_pages_back_as_they_fall_out_of_it():
    """A group with a window of 100 positions: a sequence grows to 1,000 positions in a cache of 5 pages, holds at most 3 pages
    at a time, and its table names no page that it no longer holds."""
    need = CacheNeed("kv", n_kv_heads=1, head_dim=16, window=100)
    cache = SequenceCache({"w": (need, 2)}, max_tokens=64 * 5, max_sequence_tokens=1024, dtype=torch.float32, device=torch.device("cpu"))
    assert cache.pages_per_sequence == 16 and cache.max_sequence_tokens == 1024      # not bounded by the 5 pages there are
    slot, other = cache.open(), cache.open()
    cache.reserve(other, 64)
    cache.advance(other, 64)                  # a neighbour that keeps one page throughout
    length = 0
    for step in (70, 1, 1, 50, 64, 1, 100, 13):
        for _ in range(3):
            if length + step > 1000:
                break
            assert cache.pages_needed(slot, length + step) <= cache.free_tokens() // 64
            cache.reserve(slot, length + step)
            length += step
            cache.advance(slot, length)
            cache.check()
            group = cache.kv["w"]
            first_needed = max(0, length - 100 + 1) // 64
            assert group.released[slot] == first_needed
            assert len(group.held[slot]) == -(-length // 64) - first_needed <= 3
            row = cache.page_rows("w", [slot], cache.pages_per_sequence)[0]
            assert list(row[first_needed : first_needed + len(group.held[slot])]) == group.held[slot]
            assert not row[:first_needed].any()
    cache.close(slot)
    cache.close(other)
    cache.check()
    assert cache.free_tokens() == 64 * 5


def test_groups_with_and_without_a_window_side_by_side():
    """The group without a window keeps every page (and bounds the sequence by the pages there are); the other lets go."""
    groups = {"all": (CacheNeed("kv", n_kv_heads=1, head_dim=16), 1), "w": (CacheNeed("kv", n_kv_heads=2, head_dim=32, window=64), 1)}
    cache = SequenceCache(groups, max_tokens=64 * 6, max_sequence_tokens=4096, dtype=torch.float32, device=torch.device("cpu"))
    assert cache.pages_per_sequence == 6
    slot = cache.open()
    cache.reserve(slot, 300)
    cache.advance(slot, 300)
    assert len(cache.kv["all"].held[slot]) == 5 and cache.kv["all"].released[slot] == 0
    assert len(cache.kv["w"].held[slot]) == 2 and cache.kv["w"].released[slot] == 3
    assert cache.free_tokens() == 64          # the fuller pool decides
    assert cache.live_bytes() == 300 * cache.kv["all"].bytes_per_token() + 64 * cache.kv["w"].bytes_per_token()
    cache.check()
    cache.close(slot)
    cache.check()


def test_a_cache_that_does_not_fit_is_refused_with_what_would_fit():
    """crates/engine/src/model_engine/tests/kv_budget.rs: pure arithmetic on a supplied memory snapshot."""
    from tau_rs_b200.cache.budget import CacheDoesNotFit, check_fits, headroom, kv_bytes_per_token
    from tau_rs_b200.parts.base import CacheNeed

    groups = {"kv": (CacheNeed("kv", n_kv_heads=8, head_dim=128), 36)}
    per_token = kv_bytes_per_token(groups, 2)
    assert per_token == 147456                                         # the Qwen3-8B figure
    gib = 1 << 30
    assert headroom(180 * gib) == 180 * gib // 32 and headroom(16 * gib) == 2 * gib
    assert check_fits(groups, 64 * 8192, 64, 2, 160 * gib, 180 * gib) == 64 * 8192 * per_token
    assert check_fits(groups, 100, 2, 2, 160 * gib, 180 * gib) == 128 * per_token      # whole pages
    with pytest.raises(CacheDoesNotFit) as refusal:
        check_fits(groups, 64 * 8192, 64, 2, 60 * gib, 180 * gib)
    error = refusal.value
    assert error.asked_tokens == 64 * 8192 and error.needed_bytes == 64 * 8192 * per_token and error.free_bytes == 60 * gib
    assert error.fitting_tokens % 64 == 0 and 0 < error.fitting_tokens < 64 * 8192
    assert check_fits(groups, error.fitting_tokens, 64, 2, 60 * gib, 180 * gib) > 0
    with pytest.raises(CacheDoesNotFit):
        check_fits(groups, error.fitting_tokens + 64, 64, 2, 60 * gib, 180 * gib)
    with pytest.raises(CacheDoesNotFit) as nothing:
        check_fits(groups, 64, 1, 2, 1 * gib, 180 * gib)
    assert nothing.value.fitting_tokens == 0 and "at most 0 tokens" in str(nothing.value)
    with pytest.raises(ValueError):
        check_fits(groups, 64, 1, 2, 200 * gib, 180 * gib)
    state = {"kv": groups["kv"], "s": (CacheNeed("state", state_shape=(4, 16), state_dtype=torch.float32), 3)}
    assert check_fits(state, 64, 5, 2, 160 * gib, 180 * gib, headroom_bytes=0) == 64 * per_token + 5 * 3 * 4 * 16 * 4
