"""CPU: what the request cache does when its tier refuses, fills up, closes or loses a read, through a tier whose
transfers finish when the test says so. Behaviours follow the reference's facade tests, restated on this repo's
handles for KV blocks (the reference couples them to tiered recurrent states; a cache that is not state-coupled treats
every block the way the reference treats a block a state on disk needs):
  dev/tests/engine/kv_first_cache_test.cpp:1963-1994  a refused demotion keeps the leaf while transfers land
  :1996-2015                                           a tier that takes nothing drops the leaf instead of parking it
  :2016-2049, :2053-2085                               a leaf its tier subtree hangs on stays while the tier may write,
                                                       and goes with the subtree once the tier has closed
  :2153-2181                                           a full tier is asked once, not once per leaf
  :2219-2267                                           a full quota replaces the oldest redundant copy, then the oldest
                                                       tier-only leaf
  :2350-2406                                           a failed restore drops the blocks below it
  :1736-1802                                           a cancelled request takes back the reads that were not submitted
  :2525-2568                                           a lookup keeps the resident boundary of a tier chain warm
  :1879-1910                                           (state-coupled) tails no state needs are dropped, never written
and Cache::demoteKv / freeDiskSpace / dropDiskSubtree / dropPoisoned / endRequest (runtime/engine/cache/Cache.cpp:
143-177, 629-686, 824-905)."""
import numpy as np

from richengine_b200.hostplane import DENIED, GRANTED, NO_PAGE, PENDING, Cache, KvPool


def make(pages=8, extent=8, slots=8, transfers=8):
    pool = KvPool(pages=pages + extent, bytes_per_page=100, extent_pages=extent, runway_pages=0, budget_pages=pages)
    return pool, Cache(pool, Cache.MANUAL_TIER, slots, transfers)


def prompt(seed, n=129):
    return np.random.default_rng(seed).integers(0, 50000, size=n, dtype=np.uint32)


def publish(cache, request, text, tokens):
    cache.begin_request(request)
    assert cache.ensure_tokens(request, tokens) == GRANTED
    cache.publish(request, text, tokens)
    blocks = [cache.block_at(request, 32 * (i + 1)) for i in range(tokens // 32)]
    cache.end_request(request)
    return blocks


def land(cache, success=True):
    assert cache.complete_transfer(success)
    cache.poll_transfers()


def resident(cache, blocks):
    return [cache.block_state(b)["page"] != NO_PAGE for b in blocks]


def test_a_refused_demotion_keeps_the_leaf_while_transfers_land():
    pool, cache = make()
    a, b = prompt(1), prompt(2, 65)
    chain_a, chain_b = publish(cache, 1, a, 128), publish(cache, 2, b, 64)
    cache.manual_tier_set(1)                                   # one transfer at a time
    step = cache.evict_one()
    assert step["progress"] and cache.snapshot()["demotions"] == 1 and cache.snapshot()["transfers"] == 1
    # the other chain's leaf is asked next: the tier is busy, a transfer in flight will make room, so the leaf stays
    # and the wait is reported (a's next block is no leaf while the page being written is still resident)
    step = cache.evict_one()
    assert not step["progress"] and step["pending"]
    assert cache.snapshot()["demotions"] == 1 and cache.tier_counters()["demotions_refused"] == 1
    assert pool.snapshot()["pages_prefix"] == 6 and resident(cache, chain_a + chain_b) == [True] * 6
    cache.begin_request(9)
    assert cache.ensure_tokens(9, 32 * 3) == PENDING           # two pages are free, one more is on its way
    land(cache)
    assert cache.ensure_tokens(9, 32 * 3) == GRANTED
    cache.end_request(9)
    step = cache.evict_one()                                    # now the tier has room again
    assert step["progress"] and cache.snapshot()["demotions"] == 2
    land(cache)
    cache.close(); pool.close()


def test_a_tier_that_takes_nothing_drops_the_leaf_instead_of_parking_it():
    pool, cache = make()
    chain = publish(cache, 1, prompt(1), 128)
    cache.manual_tier_set(0)
    # nothing is in flight and nothing ever makes room: waiting would be waiting for nothing
    step = cache.evict_one()
    assert step["progress"] and not step["pending"]
    assert cache.snapshot()["demotions"] == 0 and cache.tier_counters()["demotions_refused"] == 1
    assert pool.snapshot()["pages_prefix"] == 3 and cache.snapshot()["tier_blocks"] == 0
    assert len(cache.lookup(prompt(1))) == 3
    cache.begin_request(2)
    assert cache.ensure_tokens(2, 32 * 5) == GRANTED            # no request waits although nothing was in flight
    cache.end_request(2)
    cache.close(); pool.close()


def test_a_leaf_its_tier_subtree_hangs_on_stays_while_the_tier_may_write_and_goes_with_it_once_closed():
    pool, cache = make()
    text = prompt(1)
    chain = publish(cache, 1, text, 128)
    assert cache.evict_one()["progress"]
    land(cache)                                                 # the deepest block lives in the tier only
    assert resident(cache, chain) == [True, True, True, False] and cache.snapshot()["tier_blocks"] == 1
    cache.manual_tier_set(0)                                    # writable, but it takes no transfer now
    step = cache.evict_one()                                    # the new leaf is refused: erasing it would orphan the copy below
    assert not step["progress"] and resident(cache, chain) == [True, True, True, False]
    assert cache.snapshot()["tier_blocks"] == 1 and len(cache.lookup(text)) == 4
    cache.manual_tier_set(8, writable=False)                    # a failed write has closed the tier
    cache.begin_request(5)                                      # a request that holds the tier-only block keeps the subtree
    status, _ = cache.attach_prefix(5, cache.lookup(text))
    assert status == GRANTED
    other = publish(cache, 6, prompt(7, 33), 32)                # an unrelated idle leaf is what goes meanwhile
    step = cache.evict_one()
    assert step["progress"] and len(cache.lookup(prompt(7, 33))) == 0 and len(cache.lookup(text)) == 4
    land(cache)
    cache.end_request(5)
    assert cache.evict_one()["progress"]                        # the restored leaf has its copy: the page goes at once
    assert resident(cache, chain) == [True, True, True, False]
    step = cache.evict_one()                                    # block three cannot be written any more: it leaves with the
    assert step["progress"]                                     # copy that hangs on it, as without a tier
    assert cache.snapshot()["tier_blocks"] == 0 and len(cache.lookup(text)) == 2
    assert pool.snapshot()["pages_prefix"] == 2
    cache.close(); pool.close()


def test_a_full_tier_is_asked_once_not_once_per_leaf():
    pool, cache = make()
    chains = [publish(cache, r + 1, prompt(r + 1, 33), 32) for r in range(4)]   # four leaves
    cache.manual_tier_set(1)
    assert cache.evict_one()["progress"] and cache.snapshot()["demotions"] == 1
    step = cache.evict_one()      # every other leaf would hear the same answer: the scan asks once and waits
    assert not step["progress"] and step["pending"] and cache.tier_counters()["demotions_refused"] == 1
    assert pool.snapshot()["pages_prefix"] == 4
    land(cache)
    assert pool.snapshot()["pages_prefix"] == 3
    cache.close(); pool.close()


def test_a_full_quota_replaces_the_oldest_redundant_copy_then_the_oldest_tier_only_leaf():
    pool, cache = make(slots=1)
    texts = [prompt(r + 1, 33) for r in range(3)]
    a, b, c = (publish(cache, r + 1, texts[r], 32)[0] for r in range(3))
    assert cache.evict_one()["progress"]                        # A goes to the tier ...
    land(cache)
    assert cache.block_state(a)["page"] == NO_PAGE
    cache.begin_request(9)                                      # ... and comes back: RAM and tier both hold it
    assert cache.attach_prefix(9, cache.lookup(texts[0]))[0] == GRANTED
    land(cache)
    cache.end_request(9)
    state = cache.block_state(a)
    assert state["page"] != NO_PAGE and state["tier_copy"]
    # B needs the one slot: A's redundant copy goes, A stays resident
    assert cache.evict_one()["progress"] and cache.snapshot()["demotions"] == 2
    assert cache.tier_counters()["replaced_copies"] == 1
    state = cache.block_state(a)
    assert state["page"] != NO_PAGE and not state["tier_copy"] and pool.snapshot()["pages_prefix"] == 3
    land(cache)
    assert cache.block_state(b)["page"] == NO_PAGE and cache.snapshot()["tier_blocks"] == 1
    # C needs the slot: no redundant copy is left, so the oldest tier-only leaf, B, leaves
    assert cache.evict_one()["progress"] and cache.snapshot()["demotions"] == 3
    assert cache.tier_counters()["replaced_copies"] == 2
    assert len(cache.lookup(texts[1])) == 0 and len(cache.lookup(texts[0])) == 1
    land(cache)
    assert cache.block_state(c)["page"] == NO_PAGE and cache.snapshot()["tier_blocks"] == 1
    cache.close(); pool.close()


def test_a_failed_restore_drops_the_blocks_below_it():
    pool, cache = make()
    text = prompt(1)
    chain = publish(cache, 1, text, 128)
    for _ in range(3):                                          # the three deepest blocks move to the tier
        assert cache.evict_one()["progress"]
        land(cache)
    assert resident(cache, chain) == [True, False, False, False] and cache.snapshot()["tier_blocks"] == 3
    cache.begin_request(2)
    assert cache.attach_prefix(2, cache.lookup(text))[0] == GRANTED and cache.restore_status(2) == 1
    land(cache, success=False)                                  # the second block's read fails ...
    land(cache); land(cache)                                    # ... the two below it land
    assert cache.restore_status(2) == 2 and cache.snapshot()["failed_transfers"] == 1
    assert len(cache.lookup(text)) == 1                         # the chain ends above the poisoned block at once
    assert cache.snapshot()["tier_blocks"] == 2                 # the copy that failed to read is given up at once; the blocks
    assert all(cache.block_state(b) is not None for b in chain)  # stay while the request holds them
    cache.end_request(2)
    # once the request has let go, the poisoned block and everything below it leave, pages and tier slots with them
    assert cache.snapshot()["tier_blocks"] == 0 and pool.snapshot()["pages_prefix"] == 1
    assert all(cache.block_state(b) is None for b in chain[1:]) and len(cache.lookup(text)) == 1
    fresh = publish(cache, 3, text, 128)                        # the content can be published again
    assert fresh[0] == chain[0] and len(cache.lookup(text)) == 4
    cache.close(); pool.close()


def test_a_cancelled_request_takes_back_the_reads_that_were_not_submitted():
    pool, cache = make()
    text = prompt(1)
    chain = publish(cache, 1, text, 128)
    for _ in range(3):
        assert cache.evict_one()["progress"]
        land(cache)
    free_before = pool.snapshot()["pages_free"]
    cache.manual_tier_set(1)                                    # the tier takes one read at a time
    cache.begin_request(2)
    assert cache.attach_prefix(2, cache.lookup(text))[0] == GRANTED
    assert pool.snapshot()["pages_free"] == free_before - 3 and cache.snapshot()["transfers"] == 3
    cache.poll_transfers()                                      # asked once per poll: still one submitted, two queued
    cache.end_request(2)                                        # the client went away
    # the two queued reads had no IO to drain: their pages are back, the blocks are tier-only again
    assert cache.tier_counters()["cancelled_restores"] == 2 and cache.snapshot()["transfers"] == 1
    assert pool.snapshot()["pages_free"] == free_before - 1
    assert resident(cache, chain) == [True, True, False, False]
    land(cache)                                                 # the submitted read keeps its page and lands
    assert not cache.block_state(chain[1])["transferring"] and cache.snapshot()["transfers"] == 0
    assert len(cache.lookup(text)) == 4
    cache.close(); pool.close()


def test_queued_reads_start_in_block_order_and_stop_at_the_first_refusal():
    pool, cache = make(pages=16, extent=8)
    a, b = prompt(1, 97), prompt(2, 97)
    chain_a, chain_b = publish(cache, 1, a, 96), publish(cache, 2, b, 96)
    for _ in range(6):
        assert cache.evict_one()["progress"]
        land(cache)
    assert cache.snapshot()["tier_blocks"] == 6
    cache.manual_tier_set(2)                                    # two transfers in flight, of which restores at most two
    for request, text in ((3, a), (4, b)):
        cache.begin_request(request)
        assert cache.attach_prefix(request, cache.lookup(text))[0] == GRANTED
    # submitted: a's first two blocks; queued: a's third and all of b, in that order
    land(cache)
    assert not cache.block_state(chain_a[0])["transferring"]
    land(cache)
    land(cache)                                                 # a's third block went before any of b's
    assert [cache.block_state(x)["transferring"] for x in chain_a] == [False] * 3
    assert cache.restore_status(3) == 0 and cache.restore_status(4) == 1
    while cache.complete_transfer(True):
        cache.poll_transfers()
    assert cache.restore_status(4) == 0
    cache.end_request(3); cache.end_request(4)
    cache.close(); pool.close()


def test_a_lookup_keeps_the_resident_boundary_of_a_tier_chain_warm():
    pool, cache = make()
    a, b = prompt(1), prompt(2, 65)
    chain_a = publish(cache, 1, a, 128)
    chain_b = publish(cache, 2, b, 64)
    for _ in range(2):                                          # a's two deepest blocks move to the tier
        assert cache.evict_one()["progress"]
        land(cache)
    assert resident(cache, chain_a) == [True, True, False, False]
    assert len(cache.lookup(a)) == 4                            # touches the tier-only tip AND the resident boundary
    assert cache.evict_one()["progress"]                        # so b's leaf is now the coldest resident leaf
    land(cache)
    assert resident(cache, chain_a) == [True, True, False, False] and resident(cache, chain_b) == [True, False]
    cache.close(); pool.close()


def test_a_state_coupled_cache_drops_tails_no_state_needs_and_writes_what_a_state_restores_through():
    pool, cache = make()
    cache.set_state_coupled(True)
    text = prompt(1)
    chain = publish(cache, 1, text, 128)
    cache.publish_state(chain[2], 100)                          # the conversation resumes after 96 tokens
    step = cache.evict_one(pages_only=True)                     # the tail nothing restores through is dropped, never written
    assert step["progress"] and cache.snapshot()["demotions"] == 0 and pool.snapshot()["pages_prefix"] == 3
    assert len(cache.lookup(text)) == 3
    step = cache.evict_one(pages_only=True)                     # a page scan takes the state off its leaf first ...
    assert step["progress"] and step["evicted_state"]
    step = cache.evict_one(pages_only=True)                     # ... and then nothing needs the leaf any more: dropped too
    assert step["progress"] and cache.snapshot()["demotions"] == 0 and pool.snapshot()["pages_prefix"] == 2
    # with the state kept below, the leaf above it is written: the state restores through it
    cache.publish_state(chain[1], 100)
    cache.pin_state(chain[1])
    rest = publish(cache, 2, text, 128)
    assert rest[:2] == chain[:2]
    cache.unpin_state(chain[1])
    cache.publish_state(rest[3], 100)
    cache.use_state(rest[3])                                    # a running request resumes from the deepest state
    step = cache.evict_one(up_to_in_use=True, pages_only=True)
    assert step["progress"]
    cache.close(); pool.close()


def test_reclaim_for_pages_evicts_exactly_the_shortfall():
    """dev/tests/engine/kv_first_cache_test.cpp:2488-2521 (the case without states)."""
    pool = KvPool(pages=16, bytes_per_page=100, extent_pages=1, runway_pages=0, budget_pages=8)
    cache = Cache(pool, Cache.NO_TIER, 0, 0)
    for leaf in range(8):   # eight one-page leaves fill the budget
        publish(cache, leaf + 1, np.full(33, 100 + leaf, dtype=np.uint32), 32)
    assert pool.snapshot()["pages_free"] == 0 and pool.snapshot()["pages_prefix"] == 8
    assert cache.reclaim_for_pages(3) == 3
    assert pool.snapshot()["pages_free"] == 3 and pool.snapshot()["pages_prefix"] == 5
    assert cache.reclaim_for_pages(3) == 0   # nothing more once the shortfall is covered
    cache.close(); pool.close()


def test_a_restore_keeps_the_block_it_extends_and_waits_for_the_room_being_made():
    """dev/tests/engine/kv_first_cache_test.cpp:2566-2626: the lookup warmed the resident boundary, so the reclaim that
    makes room for the restore takes an older leaf; while that leaf's copy is on its way the restore is Pending and
    holds no page."""
    pool, cache = make(pages=6, extent=2)
    text, other = prompt(1), prompt(2, 65)
    chain = publish(cache, 1, text, 128)
    assert cache.evict_one()["progress"]                        # the last block goes to the tier
    land(cache)
    side = publish(cache, 2, other, 64)                         # a newer chain beside it
    cache.begin_request(3)
    assert cache.ensure_tokens(3, 32) == GRANTED                # and a request that holds the rest
    assert pool.snapshot()["pages_free"] == 0
    found = cache.lookup(text)                                  # tip and resident boundary are now the warmest blocks
    assert len(found) == 4
    cache.begin_request(4)
    assert cache.attach_prefix(4, found)[0] == DENIED           # nothing free, nothing on its way
    assert cache.reclaim_for_pages(1) == 1                      # making room demotes the OTHER chain's leaf, not the
    assert cache.block_state(side[1])["transferring"]           # block the restore extends
    assert resident(cache, chain) == [True, True, True, False]
    status, _ = cache.attach_prefix(4, found)
    assert status == PENDING and cache.page_table(4)[0] == []   # a restore without a page waits and holds none meanwhile
    land(cache)
    status, resume = cache.attach_prefix(4, found)
    assert status == GRANTED and resume == 128 and NO_PAGE not in cache.page_table(4)[0]
    land(cache)
    assert cache.restore_status(4) == 0
    cache.end_request(4); cache.end_request(3)
    cache.close(); pool.close()


def test_a_reclaim_step_returns_whole_extents_before_it_evicts():
    """dev/tests/engine/kv_first_cache_test.cpp:2858-2905 (Cache::reclaimOne with ReleaseExtents, Cache.cpp:436-449,
    692-698): an empty extent goes as it is; scattered free pages are gathered into one before anything is evicted, and
    requests and cached blocks follow the moved page; when the free pages cover no extent, the step evicts."""
    pool = KvPool(pages=16, bytes_per_page=100, extent_pages=4, runway_pages=0, budget_pages=16)
    cache = Cache(pool, Cache.NO_TIER, 0, 0)
    texts = [prompt(10 + r, 97) for r in range(3)]
    for r, text in enumerate(texts):              # nine pages over three extents, in order
        cache.begin_request(r + 1)
        assert cache.ensure_tokens(r + 1, 96) == GRANTED
        for i, page in enumerate(cache.page_table(r + 1)[0]):
            pool.set_page_content(page, 100 * r + i)
        cache.publish(r + 1, text, 96)
        cache.end_request(r + 1)
    cache.begin_request(7)                        # a request that touched a fourth extent and left
    assert cache.ensure_tokens(7, 32 * 7) == GRANTED
    cache.end_request(7)
    assert pool.snapshot()["pages_allocated"] == 16 and pool.snapshot()["pages_prefix"] == 9
    cache.begin_request(4)                        # the second prompt is in use by a request
    status, _ = cache.attach_prefix(4, cache.lookup(texts[1]))
    assert status == GRANTED
    table, revision, _ = cache.page_table(4)
    for _ in range(3):                            # the first prompt is evicted: its extent keeps one page of the second
        assert cache.evict_one()["progress"]
    assert len(cache.lookup(texts[0])) == 0 and pool.snapshot()["pages_prefix"] == 6

    step = cache.reclaim_step(Cache.RELEASE_EXTENTS)
    assert step["progress"] and step["bytes"] == 400 and pool.snapshot()["pages_allocated"] == 12   # the empty extent, as it is
    assert pool.snapshot()["extent_compactions"] == 0
    step = cache.reclaim_step(Cache.RELEASE_EXTENTS)
    snapshot = pool.snapshot()                    # scattered free pages are gathered before anything is evicted
    assert step["progress"] and step["bytes"] == 400 and not step["evicted_state"]
    assert snapshot["pages_allocated"] == 8 and snapshot["pages_prefix"] == 6 and snapshot["extent_compactions"] == 1
    moved, revision_after, first_changed = cache.page_table(4)
    assert revision_after == revision + 1 and first_changed == 0 and moved != table
    assert [pool.page_content(page) for page in moved] == [100, 101, 102]   # the request follows its moved page
    cache.end_request(4)
    cache.begin_request(5)
    status, _ = cache.attach_prefix(5, cache.lookup(texts[1]))
    assert status == GRANTED and cache.page_table(5)[0] == moved           # and so does the cached block
    cache.end_request(5)
    step = cache.reclaim_step(Cache.RELEASE_EXTENTS)   # the two free pages left cover no extent: the next step evicts
    assert step["progress"] and step["bytes"] == 0 and pool.snapshot()["pages_prefix"] == 5
    assert pool.snapshot()["extent_compactions"] == 1

    done = cache.evict_all()                       # everything unpinned goes, then every extent
    assert done["progress"] and pool.snapshot()["pages_allocated"] == 0 and pool.snapshot()["pages_prefix"] == 0
    cache.close(); pool.close()


def test_evict_all_gathers_what_requests_hold_into_one_extent():
    """dev/tests/engine/kv_first_cache_test.cpp:3019-3045 (Cache::evictAll): everything unpinned goes before anything
    moves, so no page is moved and then evicted; what a request holds ends up in one extent."""
    pool = KvPool(pages=16, bytes_per_page=100, extent_pages=4, runway_pages=0, budget_pages=16)
    cache = Cache(pool, Cache.NO_TIER, 0, 0)
    texts = [prompt(20 + r, 97) for r in range(3)]
    for r, text in enumerate(texts):
        cache.begin_request(r + 1)
        assert cache.ensure_tokens(r + 1, 96) == GRANTED
        for i, page in enumerate(cache.page_table(r + 1)[0]):
            pool.set_page_content(page, 100 * r + i)
        cache.publish(r + 1, text, 96)
        cache.end_request(r + 1)
    cache.begin_request(4)                        # the second prompt, whose pages straddle two extents, is held
    assert cache.attach_prefix(4, cache.lookup(texts[1]))[0] == GRANTED
    for _ in range(3):
        assert cache.evict_one()["progress"]     # the first prompt goes
    moves_before = pool.snapshot()["pages_moved"]
    done = cache.evict_all()
    snapshot = pool.snapshot()
    assert done["progress"] and done["bytes"] == 800                       # two of the three extents return
    assert snapshot["pages_allocated"] == 4 and snapshot["pages_prefix"] == 3 and snapshot["pages_free"] == 1
    assert snapshot["pages_moved"] - moves_before == 1                     # only the one page outside the gathered extent moved
    table = cache.page_table(4)[0]
    assert len({page // 4 for page in table}) == 1
    assert [pool.page_content(page) for page in table] == [100, 101, 102]
    assert len(cache.lookup(texts[2])) == 0 and len(cache.lookup(texts[1])) == 3
    cache.end_request(4)
    cache.close(); pool.close()


def test_compaction_leaves_pages_in_transfer_where_they_are():
    """dev/tests/engine/kv_first_cache_test.cpp:3047-3126, 3128-3210: a page a restore reads into, or a demotion reads
    from, stays put: the extent that holds it is passed over although it has the fewest pages, and the next one moves."""
    pool = KvPool(pages=16, bytes_per_page=100, extent_pages=4, runway_pages=0, budget_pages=16)
    cache = Cache(pool, Cache.MANUAL_TIER, 8, 8)
    tiered, plain, kept = prompt(31, 33), prompt(32, 97), prompt(33, 97)
    publish(cache, 1, tiered, 32)
    assert cache.evict_one()["progress"]
    land(cache)                                                  # one block lives in the tier only
    publish(cache, 2, plain, 96)                                 # three plain blocks on the first extent
    cache.begin_request(3)
    assert cache.attach_prefix(3, cache.lookup(tiered))[0] == GRANTED and cache.restore_status(3) == 1
    reading_into = cache.page_table(3)[0][0]                     # the restore takes the extent's last page and stays in flight
    assert reading_into // 4 == cache.block_state(cache.lookup(plain)[0])["page"] // 4
    cache.begin_request(4)
    assert cache.ensure_tokens(4, 96) == GRANTED
    for i, page in enumerate(cache.page_table(4)[0]):
        pool.set_page_content(page, 40 + i)
    cache.publish(4, kept, 96)
    cache.end_request(4)
    assert {cache.block_state(b)["page"] // 4 for b in cache.lookup(kept)} == {reading_into // 4 + 1}
    cache.set_state_coupled(True)                                # from here on a leaf no state needs is dropped, not written
    assert len(cache.lookup(kept)) == 3                          # the kept chain is the warmer one: the plain leaves go
    for _ in range(3):
        assert cache.evict_one()["progress"]
    assert len(cache.lookup(plain)) == 0 and len(cache.lookup(kept)) == 3 and cache.snapshot()["transfers"] == 1
    # the first extent keeps only the page being read into: it holds the fewest pages, and is passed over
    moved_before = pool.snapshot()["pages_moved"]
    assert cache.compact_extent()
    assert pool.snapshot()["pages_moved"] - moved_before == 3 and cache.page_table(3)[0][0] == reading_into
    land(cache)
    assert cache.restore_status(3) == 0 and cache.page_table(3)[0][0] == reading_into
    cache.end_request(3)
    cache.begin_request(5)
    assert cache.attach_prefix(5, cache.lookup(kept))[0] == GRANTED
    table = cache.page_table(5)[0]                               # the kept chain followed its pages, next to the restored one
    assert {page // 4 for page in table} == {reading_into // 4} and [pool.page_content(page) for page in table] == [40, 41, 42]
    cache.end_request(5)
    # the same for a page a demotion reads from
    cache.set_state_coupled(False)
    publish(cache, 6, prompt(34, 161), 160)                      # five more pages, spilling into a third extent
    cache.lookup(prompt(34, 161))
    while not cache.snapshot()["transfers"]:                     # (the restored block has its copy and goes at once)
        assert cache.evict_one()["progress"]                     # now the oldest leaf's copy is in flight
    victim = next(b for b in cache.lookup(kept) if cache.block_state(b)["transferring"])
    being_written = cache.block_state(victim)["page"]
    while cache.compact_extent():
        assert cache.block_state(victim)["page"] == being_written
    land(cache)
    assert cache.block_state(victim)["page"] == NO_PAGE
    cache.close(); pool.close()
