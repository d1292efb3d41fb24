"""CPU: the page allocator — side by side with the reference's own allocator compiled in place
(oracle/_ref), and the behaviours its tests pin (dev/tests/engine/elastic_kv_pool_test.cpp)."""
import ctypes as C

import numpy as np
import pytest

import oracle as om
from richengine_b200.hostplane import KvPool

needs_reference = pytest.mark.skipif(om.reference() is None, reason="reference checkout was not compiled here")


class ReferencePool:
    def __init__(self, pages, bytes_per_page, extent_pages, runway, budget=2 ** 62):
        self.r = om.reference()
        self.h = self.r.ref_pool_create(pages, bytes_per_page, extent_pages, runway, budget)
        assert self.h
        self.extent_pages = extent_pages

    def acquire(self, n):
        out = (C.c_uint32 * max(n, 1))()
        got = self.r.ref_pool_acquire(self.h, n, out)
        return None if got < 0 else list(out[:got])

    def retain(self, p, prefix=False): return self.r.ref_pool_retain(self.h, p, int(prefix))
    def release(self, p, prefix=False): return self.r.ref_pool_release(self.h, p, int(prefix))
    def reclaim(self, keep, limit): return self.r.ref_pool_reclaim(self.h, int(keep), limit)
    def set_budget(self, pages): self.r.ref_pool_set_budget(self.h, pages)

    def compact(self, fixed=()):
        f = np.ascontiguousarray(fixed, dtype=np.uint32)
        out = (C.c_uint32 * self.extent_pages)()
        first = self.r.ref_pool_compact(self.h, f.ctypes.data, len(f), out)
        return None if first < 0 else (first, list(out))

    def snapshot(self):
        out = (C.c_uint64 * 10)()
        self.r.ref_pool_snapshot(self.h, out)
        return list(out)

    def close(self): self.r.ref_pool_destroy(self.h)


@needs_reference
@pytest.mark.parametrize("seed", range(6))
def test_random_trace_matches_reference_pool(seed):
    """Same operations, same page ids, refusals, moves and counters."""
    rng = np.random.default_rng(seed)
    extent, extents = int(rng.choice([4, 8, 16])), int(rng.integers(3, 9))
    pages = extent * extents
    runway = int(rng.integers(0, extent + 1))
    budget = int(rng.integers(extent, pages - extent + 1))  # page ids always outnumber the budget
    mine = KvPool(pages=pages, bytes_per_page=1000, extent_pages=extent, runway_pages=runway, budget_pages=budget)
    ref = ReferencePool(pages, 1000, extent, runway, budget)
    active, prefix = {}, set()  # page -> active references; pages the cache owns
    for step in range(600):
        op = rng.choice(["acquire", "release", "retain", "prefix", "unprefix", "reclaim", "compact", "budget"],
                        p=[0.3, 0.3, 0.08, 0.08, 0.08, 0.06, 0.06, 0.04])
        if op == "acquire":
            n = int(rng.integers(1, 2 * extent))
            a, b = mine.acquire(n), ref.acquire(n)
            assert a == b, (step, n)
            for p in a or []:
                active[p] = active.get(p, 0) + 1
        elif op == "release" and active:
            p = int(rng.choice(list(active)))
            mine.release(p); assert ref.release(p) == 0
            active[p] -= 1
            if not active[p]: del active[p]
        elif op == "retain" and active:
            p = int(rng.choice(list(active)))
            mine.retain(p); assert ref.retain(p) == 0
            active[p] += 1
        elif op == "prefix" and active:
            p = int(rng.choice(list(active)))
            if p not in prefix:
                mine.retain(p, True); assert ref.retain(p, True) == 0
                prefix.add(p)
        elif op == "unprefix" and prefix:
            p = int(rng.choice(list(prefix)))
            mine.release(p, True); assert ref.release(p, True) == 0
            prefix.discard(p)
        elif op == "reclaim":
            keep, limit = bool(rng.integers(0, 2)), int(rng.integers(1, 4))
            assert mine.reclaim_empty_extents(keep, limit) == ref.reclaim(keep, limit)
        elif op == "compact":
            fixed = [int(p) for p in rng.choice(list(active), size=min(len(active), 2), replace=False)] if active and rng.random() < 0.3 else []
            a, b = mine.compact_extent(fixed), ref.compact(fixed)
            assert a == b, step
            if a:
                first, destinations = a
                moved = {first + i: d for i, d in enumerate(destinations) if d != first + i}
                active = {moved.get(p, p): n for p, n in active.items()}
                prefix = {moved.get(p, p) for p in prefix}
        elif op == "budget":
            budget = int(rng.integers(extent, pages - extent + 1))
            mine.set_budget(budget); ref.set_budget(budget)
        assert list(mine.snapshot().values()) == ref.snapshot(), step
    mine.close(); ref.close()


def test_packing_runway_refusal_and_reuse_order():
    """elastic_kv_pool_test.cpp: the runway is allocated up front, a fresh extent hands out its lowest
    page first, fuller extents fill before emptier ones, a refusal returns what it took."""
    pool = KvPool(pages=32, bytes_per_page=100, extent_pages=8, runway_pages=8, budget_pages=16)
    assert pool.snapshot()["pages_allocated"] == 8 and pool.snapshot()["extent_allocations"] == 1
    assert pool.acquire(3) == [0, 1, 2]
    assert pool.acquire(7) == [3, 4, 5, 6, 7, 8, 9]  # grows by extent 1
    assert pool.acquire(7) is None                    # the budget refuses a third extent
    snap = pool.snapshot()
    assert snap["pages_active"] == 10 and snap["pages_free"] == 6  # nothing leaked by the refusal
    pool.release(1); pool.release(5)
    assert pool.acquire(2) == [5, 1]                  # most recently freed first, fullest extent (0) first
    for p in (8, 9):
        pool.release(p)
    assert pool.snapshot()["reclaimable_bytes"] == 800
    assert pool.reclaim_empty_extents(False, 4) == 800 and pool.snapshot()["pages_allocated"] == 8
    with pytest.raises(RuntimeError):
        pool.release(9)  # a page of an unallocated extent holds no reference
    with pytest.raises(RuntimeError):
        pool.retain(9)
    pool.close()


def test_prefix_ownership_and_counts():
    pool = KvPool(pages=16, bytes_per_page=10, extent_pages=8, runway_pages=0)
    (page,) = pool.acquire(1)
    pool.retain(page, prefix_owner=True)
    with pytest.raises(RuntimeError):
        pool.retain(page, prefix_owner=True)  # one block per page
    pool.release(page)  # the request lets go; the cache still owns the page
    snap = pool.snapshot()
    assert snap["pages_active"] == 0 and snap["pages_prefix"] == 1 and snap["pages_free"] == 7
    pool.retain(page)   # a later request shares it
    pool.release(page, prefix_owner=True)
    assert pool.snapshot()["pages_free"] == 7
    pool.release(page)
    assert pool.snapshot()["pages_free"] == 8
    with pytest.raises(RuntimeError):
        pool.release(page)
    pool.close()


def test_compaction_moves_references_and_content():
    pool = KvPool(pages=24, bytes_per_page=10, extent_pages=8, runway_pages=0)
    pages = pool.acquire(20)
    for p in pages:
        pool.set_page_content(p, 1000 + p)
    for p in pages[2:8] + pages[10:16] + pages[17:20]:
        pool.release(p)  # extent 0 holds 2 pages, extent 1 holds 2, extent 2 holds 1
    moved = pool.compact_extent()
    assert moved is not None
    first, destinations = moved
    assert first == 16  # the extent with the fewest pages is emptied
    target = destinations[0]
    assert target != 16 and pool.page_content(target) == 1016
    assert pool.snapshot()["extent_compactions"] == 1 and pool.snapshot()["pages_moved"] == 1
    assert pool.reclaim_empty_extents(False, 8) == 80
    pool.release(target)
    with pytest.raises(RuntimeError):
        pool.release(16)
    assert pool.compact_extent(fixed=[pages[0], pages[8]]) is None  # both remaining extents are pinned
    pool.close()
