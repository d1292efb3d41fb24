"""CPU: composite states on KV blocks and the reclaim order they impose (engine::StateCache as far as the KV path is
coupled to it, Cache::evictOne / reclaimOldest / reclaimOneState: runtime/engine/cache/Cache.cpp:451-628,
Cache.hpp:549-556). Behaviours follow the reference's facade tests, restated on this repo's handles:
  dev/tests/engine/kv_first_cache_test.cpp:743-784  a finished request's tail KV goes before its state
  :882-895, :897-909                                 checkpoints go before older KV; an optional reclaim leaves ordinary states
  :617-633, :637-652                                 a speculative reclaim keeps the resume point; a checkpoint does not outrank it
  :654-672                                           a state goes before the KV block under it; a pinned state protects its chain
and the in-use rule of Cache.cpp:451-487 (states in use and their KV go last, only to running work)."""
import numpy as np
import pytest

from richengine_b200.hostplane import GRANTED, Cache, KvPool


def make(pages=16, extent=4, tier=Cache.NO_TIER, slots=16, transfers=8):
    pool = KvPool(pages=pages, bytes_per_page=100, extent_pages=extent, runway_pages=0, budget_pages=pages)
    return pool, Cache(pool, tier, slots, transfers)


def chain(cache, request, prompt, tokens):
    """Publishes `tokens` tokens of `prompt` for a new request; returns its block ids."""
    cache.begin_request(request)
    assert cache.ensure_tokens(request, tokens) == GRANTED
    cache.publish(request, prompt, tokens)
    return [cache.block_at(request, 32 * (i + 1)) for i in range(tokens // 32)]


PROMPT = np.arange(5000, 5000 + 161, dtype=np.uint32)


def test_finished_requests_tail_kv_goes_before_its_state():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[1], 100)  # the conversation can resume after 64 tokens
    cache.end_request(1)
    assert pool.snapshot()["pages_prefix"] == 4 and cache.state_summary()["states"] == 1
    info = [cache.state_info(b) for b in blocks]
    assert [i["kv_needed"] for i in info] == [1, 1, 0, 0]  # the state's own block and the block above it
    for remaining in (3, 2):  # the two tail leaves no state needs go first, the state stays
        step = cache.evict_one()
        assert step["progress"] and not step["evicted_state"] and step["state_bytes"] == 0
        assert pool.snapshot()["pages_prefix"] == remaining and cache.state_summary()["states"] == 1
    assert len(cache.lookup(PROMPT)) == 2  # what the state resumes through is still matchable
    step = cache.evict_one()  # now the state's block is the oldest leaf: the state goes first ...
    assert step["progress"] and step["evicted_state"] and step["state_bytes"] == 100
    assert cache.state_summary()["states"] == 0 and pool.snapshot()["pages_prefix"] == 2
    step = cache.evict_one()  # ... then its block
    assert step["progress"] and not step["evicted_state"] and pool.snapshot()["pages_prefix"] == 1
    cache.close(); pool.close()


def test_checkpoints_go_before_older_kv_and_ordinary_states():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[0], 150)                  # ordinary, oldest
    cache.publish_state(blocks[2], 200, checkpoint=True)  # disposable, newer
    cache.end_request(1)
    step = cache.evict_one()
    assert step["progress"] and step["evicted_state"] and step["state_bytes"] == 200  # the checkpoint, although newest
    assert pool.snapshot()["pages_prefix"] == 4 and cache.state_info(blocks[0])["contains"]
    # a page scan has no use for a checkpoint's buffers: it takes a dead leaf instead
    cache.publish_state(blocks[2], 200, checkpoint=True)
    step = cache.evict_one(pages_only=True)
    assert step["progress"] and not step["evicted_state"] and pool.snapshot()["pages_prefix"] == 3
    cache.close(); pool.close()


def test_optional_reclaim_leaves_ordinary_states_intact():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[0], 150)
    cache.publish_state(blocks[2], 200, checkpoint=True)
    cache.end_request(1)
    assert cache.reclaim_one_state(checkpoints_only=True)  # the checkpoint is recycled for the new publication
    summary = cache.state_summary()
    assert summary["states"] == 1 and summary["bytes"] == 150
    assert not cache.reclaim_one_state(checkpoints_only=True)  # nothing disposable is left: the ordinary state stays
    assert cache.state_summary()["states"] == 1
    assert cache.reclaim_one_state()                           # a demanded publication takes it
    assert cache.state_summary()["states"] == 0
    cache.close(); pool.close()


def test_speculative_reclaim_keeps_the_resume_point_and_its_chain():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[0], 100)
    cache.publish_state(blocks[2], 100)  # the newest ordinary state: where the conversation resumes next
    cache.end_request(1)
    assert cache.state_summary()["resume_point"] == blocks[2]
    while cache.evict_one(keep_resume_point=True)["progress"]:
        pass
    summary = cache.state_summary()
    assert summary["states"] == 1 and cache.state_info(blocks[2])["contains"]
    assert pool.snapshot()["pages_prefix"] == 3  # the chain the kept state restores through survives with it
    assert len(cache.lookup(PROMPT)) == 3
    while cache.evict_one()["progress"]:         # a demanded shrink reaches the resume point too
        pass
    assert cache.state_summary()["states"] == 0 and pool.snapshot()["pages_prefix"] == 0
    cache.close(); pool.close()


def test_a_checkpoint_does_not_outrank_the_resume_point():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[0], 100)                   # a warmed ordinary state
    cache.publish_state(blocks[2], 100, checkpoint=True)  # a newer disposable checkpoint
    cache.end_request(1)
    step = cache.evict_one(keep_resume_point=True)
    assert step["progress"] and step["evicted_state"]
    assert cache.state_info(blocks[0])["contains"] and not cache.state_info(blocks[2])["contains"]
    cache.close(); pool.close()


def test_a_pinned_state_protects_the_kv_it_restores_through():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[2], 100)
    cache.end_request(1)
    cache.pin_state(blocks[2])  # a restore is reading it
    while cache.evict_one()["progress"]:
        pass
    assert pool.snapshot()["pages_prefix"] == 3 and cache.state_summary()["states"] == 1  # only the dead tail leaf went
    cache.unpin_state(blocks[2])
    step = cache.evict_one()
    assert step["evicted_state"] and step["state_bytes"] == 100  # the state first, its block after it
    assert cache.evict_one()["progress"] and pool.snapshot()["pages_prefix"] == 2
    cache.close(); pool.close()


def test_states_in_use_and_their_kv_go_last_and_only_to_running_work():
    pool, cache = make(pages=16)
    other = np.arange(9000, 9000 + 161, dtype=np.uint32)
    a = chain(cache, 1, PROMPT, 96)
    b = chain(cache, 2, other, 96)
    cache.publish_state(a[1], 100)
    cache.publish_state(b[1], 100)
    cache.use_state(a[1])  # an unfinished request of conversation A resumes from here
    cache.end_request(1); cache.end_request(2)
    assert cache.state_info(a[1])["in_use"] and cache.state_info(a[0])["kv_needed_in_use"] and not cache.state_info(a[2])["kv_needed_in_use"]
    # an ordinary reclaim takes everything else, oldest first, and stops at what is in use
    evicted = []
    while True:
        step = cache.evict_one(up_to_in_use=False)
        if not step["progress"]:
            break
        evicted.append(step["evicted_state"])
    assert cache.state_summary()["states"] == 1 and cache.state_info(a[1])["contains"]
    assert pool.snapshot()["pages_prefix"] == 2  # A's two blocks under the state in use
    assert len(cache.lookup(PROMPT)) == 2 and cache.lookup(other) == []
    # running work may take them: the state first, then its chain
    step = cache.evict_one(up_to_in_use=True)
    assert step["progress"] and step["evicted_state"]
    cache.unuse_state(a[1])
    while cache.evict_one()["progress"]:
        pass
    assert pool.snapshot()["pages_prefix"] == 0
    cache.close(); pool.close()


def test_a_use_turns_a_checkpoint_into_an_ordinary_state_and_unuse_refreshes_it():
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[0], 10, checkpoint=True)
    cache.publish_state(blocks[1], 20)
    cache.end_request(1)
    cache.use_state(blocks[0])
    assert cache.state_info(blocks[0])["ordinary"]  # a state in use is reusable
    cache.unuse_state(blocks[0])                    # the conversation resumes there next: it is the warmest now
    assert cache.state_summary()["resume_point"] == blocks[0]
    with pytest.raises(RuntimeError):
        cache.unuse_state(blocks[0])
    with pytest.raises(RuntimeError):
        cache.publish_state(123456, 10)             # a state needs its KV block in the cache
    # a boundary republished as ordinary stays ordinary when a checkpoint is offered later
    cache.publish_state(blocks[1], 25, checkpoint=True)
    info = cache.state_info(blocks[1])
    assert info["ordinary"] and info["bytes"] == 20   # the copy that is there is reused: the same block is the same content
    cache.close(); pool.close()


def test_with_a_tier_a_needed_leaf_is_demoted_and_its_state_kept_resumable():
    """With a host tier a leaf a state needs is written out (its page returns when the copy lands); the state above it
    still finds its chain by lookup, tier blocks included."""
    pool, cache = make(tier=Cache.MANUAL_TIER)
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[3], 100)
    cache.end_request(1)
    step = cache.evict_one()      # the state at the leaf goes first (its block is the oldest leaf with a state)
    assert step["evicted_state"]
    step = cache.evict_one()      # then the leaf: a demotion
    assert step["progress"] and cache.snapshot()["transfers"] == 1
    assert pool.snapshot()["pages_prefix"] == 4  # valid until its copy lands
    assert cache.complete_transfer(True)
    cache.poll_transfers()
    assert pool.snapshot()["pages_prefix"] == 3 and len(cache.lookup(PROMPT)) == 4
    cache.close(); pool.close()


def test_a_lookup_asks_for_a_junction_only_at_a_branch_point_with_a_state_below():
    """dev/tests/engine/kv_first_cache_test.cpp:543-586: a prompt that leaves the cached chain where the chain goes on
    to a state of its own branches there; its lookup names the branch point as a junction worth a state, and once a
    state is published there the next lookup resumes from it. Not at a chain end, and not inside a tail past the
    state that holds no state."""
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[0], 100)   # resumable after 32 tokens
    cache.end_request(1)
    branch = np.concatenate([PROMPT[:64], np.full(33, 7, dtype=np.uint32)])  # leaves the chain after two pages

    def junction(prompt):
        found = cache.lookup_state(prompt, record=True)
        assert found["resume_boundary"] == 32 and found["state_block"] == blocks[0]
        cache.unpin_state(found["state_block"])
        return found["junction_boundary"]

    assert junction(PROMPT) == 0 and cache.lookup_counters()["lazy_junctions"] == 0       # a chain end
    assert junction(branch) == 0 and cache.lookup_counters()["lazy_junctions"] == 0       # a dead tail past the state
    cache.publish_state(blocks[3], 100)                                                   # the chain goes on to a state
    assert junction(branch) == 64 and cache.lookup_counters()["lazy_junctions"] == 1
    cache.publish_state(blocks[1], 100)                                                   # the junction materialises
    found = cache.lookup_state(branch)
    assert found["kv_boundary"] == 64 and found["resume_boundary"] == 64 and found["junction_boundary"] == 0
    assert found["blocks"] == blocks[:2]
    cache.unpin_state(found["state_block"])
    assert cache.lookup_counters()["kv_hit_tokens"] == 128 + 64 + 64
    cache.close(); pool.close()


def test_a_lost_reusable_state_is_told_from_one_that_never_was():
    """dev/tests/engine/kv_first_cache_test.cpp:1320-1351: a block remembers that it held a reusable state; a lookup
    that finds the KV without it reports a lost state. A dropped checkpoint is not a lost state."""
    pool, cache = make()
    blocks = chain(cache, 1, PROMPT, 128)
    cache.publish_state(blocks[3], 100)
    cache.end_request(1)
    assert cache.reclaim_one_state()                      # the state goes, its KV stays
    found = cache.lookup_state(PROMPT[:129], record=True)
    assert found["kv_boundary"] == 128 and found["state_block"] == 0 and found["lost_state"]
    cache.publish_state(blocks[3], 100)                   # published again: found, not lost
    found = cache.lookup_state(PROMPT[:129])
    assert found["state_block"] == blocks[3] and not found["lost_state"]
    cache.unpin_state(blocks[3])
    cache.publish_state(blocks[1], 100, checkpoint=True)  # a disposable checkpoint that is dropped
    assert cache.reclaim_one_state(checkpoints_only=True)
    shallow = cache.lookup_state(PROMPT[:65])
    assert shallow["state_block"] == 0 and not shallow["lost_state"]
    assert cache.lookup_counters()["lost_state_misses"] == 1
    # the state a lookup returns is pinned until the caller lets go of it: no reclaim takes it meanwhile
    found = cache.lookup_state(PROMPT[:129])
    assert found["state_block"] == blocks[3]
    assert not cache.reclaim_one_state()
    cache.unpin_state(blocks[3])
    assert cache.reclaim_one_state()
    cache.close(); pool.close()


# ---- the scheduling probe (Cache::probe / Cache::refresh, runtime/engine/cache/Cache.cpp:210-234) ----------------
# Behaviours follow dev/tests/engine/kv_first_cache_test.cpp:236-254 (a probe changes no policy), :256-273 (a valid
# probe preserves lookup and accounting), :275-352 (a refresh follows the graph), :355-405 (an evicted state or block
# is not reused; a cold probe hides nothing published later), :440-452 (another cache's probe).

ASKED = PROMPT[:129]   # four full pages and the one token that is always left to recompute


def hashed(cache):
    return cache.lookup_counters()["probe_hashed_blocks"]


def test_a_probe_changes_no_policy():
    pool, cache = make()
    blocks = chain(cache, 1, ASKED, 128)
    cache.end_request(1)
    probe = cache.probe(ASKED)
    assert probe.cached_tokens == 0 and probe.matched_blocks == 4  # KV without a state is no reusable work
    cache.publish_state(blocks[0], 100)
    cache.publish_state(blocks[3], 100)
    short, full = cache.probe(ASKED[:33]), cache.probe(ASKED)
    assert short.cached_tokens == 32 and full.cached_tokens == 128
    counters = cache.lookup_counters()
    assert counters["kv_hit_tokens"] == 0 and not cache.state_info(blocks[3])["in_use"]  # no hit counted, nothing pinned
    # the probes did not refresh the oldest state's eviction order: it is still the first to go
    assert cache.reclaim_one_state()
    assert cache.probe(ASKED[:33]).cached_tokens == 0 and cache.probe(ASKED).cached_tokens == 128
    cache.close(); pool.close()


def test_a_current_probe_preserves_lookup_and_accounting():
    pool, cache = make()
    blocks = chain(cache, 1, ASKED, 128)
    cache.end_request(1)
    cache.publish_state(blocks[0], 100)
    cache.publish_state(blocks[2], 100)
    probe = cache.probe(ASKED)
    assert probe.cached_tokens == 96 and cache.lookup_counters()["kv_hit_tokens"] == 0
    before = hashed(cache)
    found = cache.lookup_state(ASKED, record=True, probe=probe)
    assert found["blocks"] == blocks and found["kv_boundary"] == 128 and found["resume_boundary"] == 96
    assert found["junction_boundary"] == 0 and found["state_block"] == blocks[2]
    counters = cache.lookup_counters()
    assert counters["kv_hit_tokens"] == 128 and counters["lazy_junctions"] == 0 and hashed(cache) == before
    cache.unpin_state(blocks[2])
    cache.close(); pool.close()


def test_a_refresh_follows_the_states_without_hashing():
    pool, cache = make()
    blocks = chain(cache, 1, ASKED, 128)
    cache.end_request(1)
    cache.publish_state(blocks[1], 100)
    probe = cache.probe(ASKED)
    assert probe.cached_tokens == 64 and hashed(cache) == 4
    cache.publish_state(blocks[3], 100)   # states come and go without a change of the block graph
    probe.refresh(ASKED)
    assert probe.cached_tokens == 128 and hashed(cache) == 4
    assert cache.reclaim_one_state() and cache.reclaim_one_state()
    probe.refresh(ASKED)
    assert probe.cached_tokens == 0 and hashed(cache) == 4
    cache.close(); pool.close()


def test_a_refresh_hashes_only_past_the_first_block_that_went():
    pool, cache = make()
    blocks = chain(cache, 1, ASKED, 128)
    cache.end_request(1)
    cache.publish_state(blocks[2], 100)
    probe = cache.probe(ASKED)
    assert probe.cached_tokens == 96 and hashed(cache) == 4
    step = cache.evict_one()   # the tail block no state needs goes (no tier: it is forgotten)
    assert step["progress"] and not step["evicted_state"] and pool.snapshot()["pages_prefix"] == 3
    # a stale probe is ignored by a lookup: it hashes the prompt itself and finds what is there now
    stale = cache.lookup_state(ASKED, probe=probe)
    assert stale["kv_boundary"] == 96
    cache.unpin_state(blocks[2])
    probe.refresh(ASKED)      # three blocks stay without hashing, one page past them is tried
    assert probe.cached_tokens == 96 and probe.matched_blocks == 3 and hashed(cache) == 5
    probed, fresh = cache.lookup_state(ASKED, probe=probe), cache.lookup_state(ASKED)
    assert probed["kv_boundary"] == fresh["kv_boundary"] == 96 and probed["resume_boundary"] == fresh["resume_boundary"] == 96
    cache.unpin_state(blocks[2]); cache.unpin_state(blocks[2])
    # the tail comes back, written by a request that continues the chain
    cache.begin_request(2)
    status, resume = cache.attach_prefix(2, probed["blocks"])
    assert status == GRANTED and resume == 96 and cache.ensure_tokens(2, 128) == GRANTED
    cache.publish(2, ASKED, 128)
    cache.end_request(2)
    probe.refresh(ASKED)
    assert hashed(cache) == 6 and probe.matched_blocks == 4    # only the page that came back was hashed
    found = cache.lookup_state(ASKED, probe=probe)
    assert found["kv_boundary"] == 128
    cache.unpin_state(blocks[2])
    cache.close(); pool.close()


def test_a_refresh_does_not_match_through_a_poisoned_block():
    pool, cache = make(pages=8, extent=8, tier=Cache.MANUAL_TIER, slots=8, transfers=4)
    blocks = chain(cache, 1, ASKED, 128)
    cache.end_request(1)
    for _ in range(2):   # the two deepest blocks move to the tier
        assert cache.reclaim_one() and cache.complete_transfer(True)
        cache.poll_transfers()
    assert [cache.block_state(b)["page"] == 0xffffffff for b in blocks] == [False, False, True, True]
    cache.publish_state(blocks[3], 100)
    probe = cache.probe(ASKED)
    assert probe.cached_tokens == 128 and probe.matched_blocks == 4
    cache.begin_request(2)
    assert cache.attach_prefix(2, cache.lookup(ASKED))[0] == GRANTED
    assert cache.complete_transfer(False)   # the third block's read fails: it is poisoned ...
    cache.poll_transfers()
    while cache.complete_transfer(True):    # ... while whatever else was started lands
        cache.poll_transfers()
    before = hashed(cache)
    probe.refresh(ASKED)
    assert probe.matched_blocks == 2 and probe.cached_tokens == 0 and hashed(cache) == before + 1
    found = cache.lookup_state(ASKED, probe=probe)
    assert found["kv_boundary"] == 64
    cache.end_request(2)
    cache.close(); pool.close()


def test_a_probe_reuses_neither_an_evicted_state_nor_an_evicted_block_and_hides_nothing_new():
    pool, cache = make()
    blocks = chain(cache, 1, ASKED, 128)
    cache.end_request(1)
    cache.publish_state(blocks[3], 100)
    probe = cache.probe(ASKED)
    assert probe.cached_tokens == 128 and cache.reclaim_one_state()
    found = cache.lookup_state(ASKED, probe=probe)   # the chain is current, the state is looked up again
    assert found["kv_boundary"] == 128 and found["state_block"] == 0 and found["resume_boundary"] == 0
    assert cache.evict_one()["progress"]              # now a block goes: the probe is stale and ignored
    assert cache.lookup_state(ASKED, probe=probe)["kv_boundary"] == 96
    # a probe taken while nothing was cached hides nothing published later
    other = np.arange(90000, 90000 + 97, dtype=np.uint32)
    cold = cache.probe(other)
    assert cold.cached_tokens == 0 and cold.matched_blocks == 0
    published = chain(cache, 2, other, 96)
    cache.publish_state(published[1], 100)
    cache.end_request(2)
    found = cache.lookup_state(other, probe=cold)
    assert found["kv_boundary"] == 96 and found["resume_boundary"] == 64
    cache.unpin_state(published[1])
    cold.refresh(other)
    assert cold.cached_tokens == 64 and cold.matched_blocks == 3
    cache.close(); pool.close()


def test_another_caches_probe_is_ignored_by_a_lookup_and_refused_by_a_refresh():
    pool_a, cache_a = make()
    pool_b, cache_b = make()
    first = np.arange(100, 100 + 65, dtype=np.uint32)
    second = np.arange(700, 700 + 65, dtype=np.uint32)
    chain(cache_a, 1, first, 64); cache_a.end_request(1)
    chain(cache_b, 1, second, 64); cache_b.end_request(1)   # the same block ids, other content
    probe = cache_a.probe(first)
    assert probe.matched_blocks == 2
    assert cache_b.lookup_state(first, probe=probe)["kv_boundary"] == 0
    with pytest.raises(RuntimeError, match="another cache"):
        probe.refresh(first, cache=cache_b)
    probe.close()
    cache_a.close(); pool_a.close(); cache_b.close(); pool_b.close()
