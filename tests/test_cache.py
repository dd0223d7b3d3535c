"""The cache's bookkeeping (no GPU): no slot or page is lost, held twice or freed twice; groups have storage of
their own; a windowed group gives pages back while the sequence runs."""
import random

import pytest

from etalii.dllm_b200.cache.allocators import CacheError, FreeList
from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache


def test_free_list_take_give_reuse():
    pool = FreeList(4, "page")
    a = pool.take(3)
    assert sorted(a) == [0, 1, 2] and pool.free == 1 and pool.held == 3
    pool.give([a[1]])
    assert pool.take(1) == [a[1]]  # what was given back last is used again first
    with pytest.raises(CacheError, match="out of pages"):
        pool.take(2)
    pool.give(a)
    with pytest.raises(CacheError, match="released twice"):
        pool.give([a[0]])
    with pytest.raises(CacheError, match="does not exist"):
        pool.give([9])
    pool.check()


def _cache(**kwargs):
    needs = [CacheNeed("kv", 2, 16), CacheNeed("kv", 2, 16), CacheNeed("kv", 1, 32, window=100), None,
             CacheNeed("state", state_shape=(3, 4))]
    return PagedCache(needs, max_tokens=64 * 20, max_length=640, device=None, **kwargs)


def test_groups_have_storage_of_their_own():
    cache = _cache()
    groups = cache.groups()
    assert [entries for _, entries in groups] == [[0, 1], [2]]
    assert groups[1][0].window == 100
    assert cache.n_pages == 20 and cache.max_pages == 10 and cache.page_size == 64


def test_sizes_from_max_tokens():
    cache = PagedCache([CacheNeed("kv", 1, 8)], max_tokens=130, max_length=10_000, device=None)
    assert cache.n_pages == 3 and cache.max_pages == 3 and cache.n_slots == 3


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    cache = _cache()
    live: dict[int, int] = {}
    for _ in range(3000):
        action = rng.random()
        try:
            if action < 0.25 and cache.slots.free:
                live[cache.acquire(1)[0]] = 0
            elif action < 0.85 and live:
                slot = rng.choice(list(live))
                n = rng.choice([1, 1, 1, 7, 64, 65, 130])
                cache.reserve(slot, n)
                cache.advance(slot, n)
                live[slot] += n
                assert cache.length(slot) == live[slot]
            elif live:
                slot = rng.choice(list(live))
                cache.release([slot])
                del live[slot]
        except CacheError as error:  # out of pages or too long: the request is refused, the books stay right
            assert "out of page" in str(error) or "exceeds" in str(error)
        cache.check()
        full = sum(-(-n // 64) for n in live.values())
        assert cache._groups[0].pool.held >= full  # the full group holds every page of every live sequence
    cache.release(list(live))
    cache.check()
    assert cache.pages_held() == 0 and cache.slots.held == 0


def test_windowed_group_returns_pages_early():
    cache = _cache()
    slot = cache.acquire(1)[0]
    for _ in range(600):
        cache.reserve(slot, 1)
        cache.advance(slot, 1)
    full, windowed = cache._groups
    assert full.pool.held == 10                 # 600 tokens in pages of 64
    assert windowed.pool.held <= 3              # a window of 100 spans at most 3 pages
    kept = [i for i, p in enumerate(windowed.pages_of[slot]) if p is not None]
    assert kept[0] * 64 <= 600 - 100 and kept[-1] == 9
    cache.release([slot])
    cache.check()
    assert cache.pages_held() == 0


def test_errors():
    cache = _cache()
    with pytest.raises(CacheError, match="not in use"):
        cache.reserve(0, 1)
    slot = cache.acquire(1)[0]
    with pytest.raises(CacheError, match="exceeds"):
        cache.reserve(slot, 641)
    cache.release([slot])
    with pytest.raises(CacheError, match="released twice"):
        cache.release([slot])
    with pytest.raises(CacheError, match="out of slots"):
        cache.acquire(cache.n_slots + 1)
    cache.check()


def test_a_released_slot_starts_again_from_zero():
    cache = _cache()
    slot = cache.acquire(1)[0]
    cache.reserve(slot, 70)
    cache.advance(slot, 70)
    pages = [p for p in cache._groups[0].pages_of[slot]]
    cache.release([slot])
    again = cache.acquire(1)[0]
    assert again == slot and cache.length(again) == 0
    cache.reserve(again, 1)
    assert cache._groups[0].pages_of[again][0] in pages  # the same storage is used again


def test_a_windowed_group_has_room_for_a_whole_prompt_of_several_windows():
    """A windowed group keeps only the window per sequence while it decodes, but a whole prompt enters in one step
    and needs all its positions at once: with a single slot and a window of 100, a prompt of 500 tokens must still
    find its pages in the windowed pool, and the planner counts with the smallest pool."""
    from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
    from etalii.dllm_b200.engine.generate import plan_batches

    cache = PagedCache([CacheNeed("kv", 2, 16, window=100), CacheNeed("kv", 2, 16)], max_tokens=64 * 40,
                       max_length=1024, dtype=None, device=None, max_slots=1)
    slot = cache.acquire(1)[0]
    cache.reserve(slot, 500)       # eight pages in both groups at once
    cache.advance(slot, 500)
    held_after_prompt = cache.pages_held()
    for _ in range(200):           # decoding: the windowed group gives pages behind the window back
        cache.reserve(slot, 1)
        cache.advance(slot, 1)
    cache.check()
    assert cache.pages_held() < held_after_prompt + 4
    assert cache.smallest_pool() < cache.n_pages
    assert plan_batches([900, 900], 50, 1024, 64, cache.smallest_pool(), 4) == [[0], [1]]
    cache.release([slot])
    cache.check()
    assert cache.pages_held() == 0
