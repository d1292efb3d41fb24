"""CPU: request page lists, prefix sharing, copy-on-write fork, truncation and eviction through a tier
whose transfers finish when the test says so. Behaviours pinned by the reference's facade tests
(dev/tests/engine/kv_first_cache_test.cpp:459-541) and block-graph tests (kv_page_cache_test.cpp),
plus the two extensions (fork, truncate)."""
import numpy as np
import pytest

from richengine_b200.hostplane import DENIED, GRANTED, NO_PAGE, PENDING, Cache, KvPool


def make(pages=64, extent=8, budget=64, tier=Cache.NO_TIER, slots=16, transfers=8):
    pool = KvPool(pages=pages + extent, bytes_per_page=100, extent_pages=extent, runway_pages=0, budget_pages=budget)
    return pool, Cache(pool, tier, slots, transfers)


def tokens(n, seed=0):
    return np.random.default_rng(seed).integers(0, 50000, size=n, dtype=np.uint32)


def test_page_table_revisions():
    """revision bumps on every change; the list equals the previous one below firstChanged
    (kv_first_cache_test.cpp:459-507)."""
    pool, cache = make()
    cache.begin_request(1)
    with pytest.raises(RuntimeError):
        cache.begin_request(1)
    with pytest.raises(RuntimeError):
        cache.begin_request(0)
    pages, revision, first = cache.page_table(1)
    assert pages == [] and revision == 0
    assert cache.ensure_tokens(1, 33) == GRANTED
    pages, revision, first = cache.page_table(1)
    assert len(pages) == 2 and revision == 1 and first == 0
    assert cache.ensure_tokens(1, 40) == GRANTED  # already covered: no change
    assert cache.page_table(1)[1] == 1
    assert cache.ensure_tokens(1, 32 * 5) == GRANTED
    pages2, revision, first = cache.page_table(1)
    assert pages2[:2] == pages and len(pages2) == 5 and revision == 2 and first == 2
    cache.end_request(1)
    assert pool.snapshot()["pages_active"] == 0
    cache.end_request(1)  # ending twice is harmless
    cache.close(); pool.close()


def test_publish_dedupes_onto_the_shared_page():
    """Identical content published by a second request swaps it onto the first one's page
    (Cache.cpp:310-332; kv_first_cache_test.cpp:481-494)."""
    pool, cache = make()
    t = tokens(100)
    for r in (1, 2):
        cache.begin_request(r)
        assert cache.ensure_tokens(r, 100) == GRANTED
    cache.publish(1, t, 70)  # two full pages
    assert cache.snapshot()["resident_blocks"] == 2 and pool.snapshot()["pages_prefix"] == 2
    before, rev_before, _ = cache.page_table(2)
    cache.publish(2, t, 96)  # three full pages; the first two exist already
    after, rev_after, first = cache.page_table(2)
    shared = cache.page_table(1)[0][:2]
    assert after[:2] == shared and after[2:] == before[2:]
    assert rev_after == rev_before + 2 and first == 1   # one swap per page, the last at index 1
    assert cache.snapshot()["resident_blocks"] == 3
    snap = pool.snapshot()
    assert snap["pages_active"] == 4 + 4 - 2            # the writer's two copies went back
    with pytest.raises(RuntimeError):
        cache.publish(2, t, 40)                          # history cannot move backwards
    with pytest.raises(RuntimeError):
        cache.publish(2, t[:50], 64)                     # committed beyond the exact tokens
    cache.end_request(1); cache.end_request(2)
    assert pool.snapshot()["pages_active"] == 0 and pool.snapshot()["pages_prefix"] == 3  # the cache keeps them
    cache.close()
    assert pool.snapshot()["pages_prefix"] == 0
    pool.close()


def test_lookup_leaves_one_token_to_recompute():
    """A prompt of n tokens matches at most (n-1)/32 pages: 31/32/33-token back-off
    (Cache.cpp:183-184; kv_first_cache_test.cpp:531-541)."""
    pool, cache = make()
    t = tokens(200, seed=3)
    cache.begin_request(1)
    assert cache.ensure_tokens(1, 200) == GRANTED
    cache.publish(1, t, 200)  # 6 full pages
    assert len(cache.lookup(t[:31])) == 0 and len(cache.lookup(t[:32])) == 0 and len(cache.lookup(t[:33])) == 1
    assert len(cache.lookup(t[:64])) == 1 and len(cache.lookup(t[:65])) == 2 and len(cache.lookup(t)) == 6
    other = t.copy(); other[40] += 1
    assert len(cache.lookup(other)) == 1  # the chain stops at the first differing page
    assert cache.lookup(np.array([], dtype=np.uint32)) == []
    cache.end_request(1); cache.close(); pool.close()


def test_prefix_sharing_refcounts_32_requests():
    """32 requests share one 8K-token prefix = 256 refcounted pages (BASELINE config 3)."""
    pool, cache = make(pages=2048, extent=128, budget=2048)
    prefix = tokens(8192 + 1, seed=5)
    cache.begin_request(1)
    assert cache.ensure_tokens(1, 8192) == GRANTED
    cache.publish(1, prefix, 8192)
    blocks = cache.lookup(prefix)
    assert len(blocks) == 256
    base = pool.snapshot()["pages_active"]
    for r in range(2, 34):
        cache.begin_request(r)
        status, resume = cache.attach_prefix(r, blocks)
        assert status == GRANTED and resume == 8192
        assert cache.page_table(r)[0] == cache.page_table(1)[0][:256]
        assert cache.ensure_tokens(r, 8192 + 512) == GRANTED  # its own 16 pages to diverge into
    snap = pool.snapshot()
    assert snap["pages_active"] == base + 32 * 16 and snap["pages_prefix"] == 256
    assert not cache.reclaim_one()  # every block is in use: nothing is evictable
    for r in range(1, 34):
        cache.end_request(r)
    assert pool.snapshot()["pages_active"] == 0 and pool.snapshot()["pages_prefix"] == 256
    cache.close(); pool.close()


def test_fork_copies_only_the_partial_tail_page():
    pool, cache = make()
    cache.begin_request(1)
    assert cache.ensure_tokens(1, 32 * 3 + 10) == GRANTED
    parent = cache.page_table(1)[0]
    for i, p in enumerate(parent):
        pool.set_page_content(p, 500 + i)
    cache.begin_request(2)
    assert cache.fork(1, 2, 32 * 3 + 10) == 1
    child = cache.page_table(2)[0]
    assert child[:3] == parent[:3] and child[3] != parent[3]
    assert pool.page_content(child[3]) == 503          # the tail page's content travelled
    assert cache.snapshot()["fork_copies"] == 1
    cache.begin_request(3)
    assert cache.fork(1, 3, 64) == 0                   # page-aligned fork point: nothing to copy
    assert cache.page_table(3)[0] == parent[:2]
    cache.end_request(1)                               # shared pages stay alive for the children
    assert pool.snapshot()["pages_active"] == 3 + 1 + 0
    with pytest.raises(RuntimeError):
        cache.fork(2, 3, 10)                           # the target already has pages
    cache.end_request(2); cache.end_request(3)
    assert pool.snapshot()["pages_active"] == 0
    cache.close(); pool.close()


def test_truncate_releases_the_rejected_tail():
    pool, cache = make(pages=4096, extent=128, budget=4096)
    cache.begin_request(1)
    committed = 65500
    assert cache.ensure_tokens(1, committed + 16 + 64) == GRANTED
    before = len(cache.page_table(1)[0])
    released = cache.truncate(1, committed + 5, 15)    # 5 of 16 accepted; 15 scratch tokens stay covered
    pages, revision, first = cache.page_table(1)
    assert len(pages) == (committed + 5 + 15 + 31) // 32 and released == before - len(pages) and first == len(pages)
    assert cache.truncate(1, committed + 5, 15) == 0
    t = tokens(committed + 5, seed=9)
    cache.publish(1, t, committed + 5)
    with pytest.raises(RuntimeError):
        cache.truncate(1, 100, 0)                       # published pages cannot be cut
    cache.end_request(1); cache.close(); pool.close()


def test_eviction_oldest_idle_leaf_through_the_tier():
    """Victims are idle leaves, oldest first; the page stays valid until the copy lands; a failed
    demotion keeps it; restores run root first; a failed restore poisons the block
    (Cache.cpp:507-550,824-851,933-1021; KvCache.cpp:577-592)."""
    pool, cache = make(pages=16, extent=8, budget=16, tier=Cache.MANUAL_TIER, slots=8, transfers=4)
    a, b = tokens(97, seed=1), tokens(97, seed=2)
    for r, t in ((1, a), (2, b)):
        cache.begin_request(r)
        assert cache.ensure_tokens(r, 96) == GRANTED
        for i, p in enumerate(cache.page_table(r)[0]):
            pool.set_page_content(p, r * 100 + i)
        cache.publish(r, t, 96)
        cache.end_request(r)
    assert pool.snapshot()["pages_prefix"] == 6 and pool.snapshot()["pages_free"] == 2  # one extent allocated so far
    chain_a = cache.lookup(a)          # touches a's tip: b is now the colder chain
    assert len(chain_a) == 3
    chain_b_before = [s["page"] for s in map(cache.block_state, range(4, 7))]
    assert cache.reclaim_one()         # demotes b's leaf (block 6)
    state = cache.block_state(6)
    assert state["transferring"] and state["page"] != NO_PAGE and pool.snapshot()["pages_prefix"] == 6
    assert cache.reclaim_one()         # demotions take at most half of the transfers: second one starts
    assert not cache.reclaim_one()     # the third must wait
    cache.begin_request(9)
    assert cache.ensure_tokens(9, 32 * 12) == PENDING  # ten pages are free, two are on their way out
    assert cache.complete_transfer(True)
    cache.poll_transfers()
    state = cache.block_state(6)
    assert state["page"] == NO_PAGE and state["tier_copy"] and pool.snapshot()["pages_prefix"] == 5
    assert cache.complete_transfer(False)              # the second demotion fails: its page stays
    cache.poll_transfers()
    assert cache.snapshot()["failed_transfers"] == 1 and pool.snapshot()["pages_prefix"] == 5
    assert cache.ensure_tokens(9, 32 * 12) == DENIED   # nothing is on its way any more
    assert cache.ensure_tokens(9, 32 * 11) == GRANTED
    cache.end_request(9)
    # b's chain is found again; its host-only leaf takes a fresh page and restores
    chain_b = cache.lookup(b)
    assert chain_b == [4, 5, 6]
    cache.begin_request(3)
    status, resume = cache.attach_prefix(3, chain_b)
    assert status == GRANTED and resume == 96 and cache.restores_pending(3)
    restored_page = cache.page_table(3)[0][2]
    assert cache.complete_transfer(True)
    cache.poll_transfers()
    assert not cache.restores_pending(3) and pool.page_content(restored_page) == 202   # b's third page is back
    cache.end_request(3)
    cache.close(); pool.close()


def test_failed_restore_poisons_the_block():
    pool, cache = make(pages=8, extent=8, budget=8, tier=Cache.MANUAL_TIER, slots=4, transfers=4)
    a = tokens(65, seed=4)
    cache.begin_request(1)
    assert cache.ensure_tokens(1, 64) == GRANTED
    cache.publish(1, a, 64)
    cache.end_request(1)
    assert cache.reclaim_one() and cache.complete_transfer(True)
    cache.poll_transfers()
    chain = cache.lookup(a)
    assert len(chain) == 2 and cache.block_state(chain[1])["page"] == NO_PAGE
    cache.begin_request(2)
    assert cache.attach_prefix(2, chain)[0] == GRANTED
    assert cache.complete_transfer(False)
    cache.poll_transfers()
    assert cache.snapshot()["failed_transfers"] == 1
    assert len(cache.lookup(a)) == 1   # the poisoned block matches nothing any more
    cache.end_request(2); cache.close(); pool.close()


def test_no_tier_evicts_by_forgetting_and_denies_when_nothing_is_evictable():
    pool, cache = make(pages=8, extent=8, budget=8)
    a = tokens(129, seed=6)
    cache.begin_request(1)
    assert cache.ensure_tokens(1, 128) == GRANTED
    cache.publish(1, a, 128)
    cache.begin_request(2)
    assert cache.ensure_tokens(2, 32 * 5) == DENIED      # 4 free pages, request 1 holds its chain
    assert cache.reclaim_for_pages(5) == 0
    cache.end_request(1)
    assert cache.reclaim_for_pages(5) == 1               # one leaf forgotten frees the fifth page
    assert cache.ensure_tokens(2, 32 * 5) == GRANTED
    assert len(cache.lookup(a)) == 3
    cache.end_request(2); cache.close(); pool.close()


def test_compaction_repoints_requests_and_blocks():
    pool, cache = make(pages=24, extent=8, budget=24)
    t = tokens(33 * 32, seed=8)
    cache.begin_request(1)
    assert cache.ensure_tokens(1, 20 * 32) == GRANTED
    pages = cache.page_table(1)[0]
    for i, p in enumerate(pages):
        pool.set_page_content(p, 7000 + i)
    cache.publish(1, t, 20 * 32)
    assert cache.truncate(1, 20 * 32, 0) == 0
    cache.end_request(1)
    for _ in range(13):                                   # forget the 13 coldest leaves: 7 blocks remain, over 1 extent
        assert cache.reclaim_one()
    cache.begin_request(2)
    status, resume = cache.attach_prefix(2, cache.lookup(t[: 7 * 32 + 1]))
    assert status == GRANTED and resume == 7 * 32
    assert cache.ensure_tokens(2, 18 * 32) == GRANTED     # spreads over the other extents
    assert cache.truncate(2, 7 * 32, 32) > 0              # and gives most of them back: fragmented pool
    before = cache.page_table(2)
    moved = cache.compact_extent()
    after = cache.page_table(2)
    if moved:
        assert after[1] == before[1] + 1 and len(after[0]) == len(before[0])
        for i, p in enumerate(after[0][:7]):
            assert pool.page_content(p) == 7000 + i       # shared prefix pages kept their content through the move
            assert cache.block_state(i + 1)["page"] == p
    cache.end_request(2); cache.close(); pool.close()
