"""CPU: the request cache side by side with the reference's OWN facade (runtime/engine/cache/Cache.cpp, KvCache.cpp,
StateCache.cpp and KvPool.cpp compiled in place into oracle/_ref, over the reference's test tier,
dev/tests/engine/TestKvTier.hpp). Random traces of the operations a scheduler issues run on both; after every step the
page tables, admissions, lookups (KV boundary, state, resume and junction boundary, lost state), reclaim outcomes and
the counters of pool, states and tier must agree. This repository's cache runs state-coupled here (a chain resumes only
through a composite state, as in the reference's hybrid model) with states that are byte counts in RAM."""
import ctypes as C

import numpy as np
import pytest

import oracle as om
from richengine_b200.hostplane import GRANTED, Cache, KvPool, image_spans

reference = om.reference()
pytestmark = pytest.mark.skipif(reference is None or not hasattr(reference, "ref_cache_create"),
                                reason="the reference's cache facade was not compiled here")


class Theirs:
    def __init__(self, pages, extent, runway, budget, tier, slots, transfers):
        self.r = reference
        self.h = self.r.ref_cache_create(pages, 100, extent, runway, budget, int(tier), slots, transfers)
        assert self.h
        self.pins = {}

    def close(self): self.r.ref_cache_destroy(self.h)
    def begin(self, request): assert self.r.ref_cache_begin(self.h, request) == 0
    def end(self, request): assert self.r.ref_cache_end(self.h, request) == 0
    def ensure(self, request, tokens): return self.r.ref_cache_ensure(self.h, request, tokens)

    def table(self, request):
        pages = (C.c_uint32 * 64)()
        revision, first = C.c_uint64(), C.c_uint32()
        count = self.r.ref_cache_page_table(self.h, request, pages, 64, C.byref(revision), C.byref(first))
        assert count >= 0
        return list(pages[:count]), revision.value, first.value

    def publish(self, request, tokens, committed, images=None):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        spans, n = image_spans(images)
        assert self.r.ref_cache_publish(self.h, request, t.ctypes.data, len(t), committed, spans.ctypes.data if n else None, n) == 0

    def block_at(self, request, boundary): return self.r.ref_cache_block_at(self.h, request, boundary)

    def lookup(self, prompt, record=False, hold=False, attach_to=0, probe=None, images=None):
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = (C.c_uint64 * 7)()
        spans, n = image_spans(images)
        assert self.r.ref_cache_lookup(self.h, t.ctypes.data, len(t), int(record), int(hold), attach_to, out, probe,
                                       spans.ctypes.data if n else None, n) == 0
        found = dict(zip(["kv_boundary", "state_block", "resume_boundary", "junction_boundary", "lost_state"], [int(x) for x in out[:5]]))
        found["lost_state"] = bool(found["lost_state"])
        return found, int(out[5]), int(out[6])

    def attach(self, request, prompt, images=None):
        found, _, status = self.lookup(prompt, attach_to=request, images=images)
        return status, found

    def pin(self, prompt, images=None):
        found, handle, _ = self.lookup(prompt, hold=True, images=images)
        if found["state_block"]:
            self.pins.setdefault(found["state_block"], []).append(handle)
        else:
            self.r.ref_cache_release_lookup(self.h, handle)
        return found["state_block"]

    def unpin(self, block): self.r.ref_cache_release_lookup(self.h, self.pins[block].pop())

    def probe(self, prompt, images=None):
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        spans, n = image_spans(images)
        handle = self.r.ref_cache_probe_create(self.h, t.ctypes.data, len(t), spans.ctypes.data if n else None, n)
        assert handle
        return handle

    def probe_refresh(self, handle, prompt, images=None):
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        spans, n = image_spans(images)
        assert self.r.ref_cache_probe_refresh(self.h, handle, t.ctypes.data, len(t), spans.ctypes.data if n else None, n) == 0

    def probe_tokens(self, handle): return self.r.ref_cache_probe_cached_tokens(handle)
    def probe_close(self, handle): self.r.ref_cache_probe_destroy(handle)
    def restore_status(self, request): return self.r.ref_cache_restore_status(self.h, request)
    def publish_state(self, block, size, checkpoint): assert self.r.ref_cache_publish_state(self.h, block, size, int(checkpoint)) == 0
    def use(self, block, on): assert self.r.ref_cache_use_state(self.h, block, int(on)) == 0

    def publish_stored(self, block, size, checkpoint):
        assert self.r.ref_cache_publish_state_stored(self.h, block, size, int(checkpoint)) == 0
        self.poll()   # retires the write that landed at once

    def evict_one(self, up_to_in_use, keep_resume_point, pages_only):
        out = (C.c_uint64 * 4)()
        assert self.r.ref_cache_evict_one(self.h, int(up_to_in_use), int(keep_resume_point), int(pages_only), out) == 0
        return {"progress": int(out[0]), "pending": int(out[1]), "evicted_state": int(out[2])}

    def reclaim_step(self, mode, up_to_in_use, keep_resume_point, keep_runway):
        out = (C.c_uint64 * 4)()
        assert self.r.ref_cache_reclaim_step(self.h, mode, int(up_to_in_use), int(keep_resume_point), int(keep_runway), out) == 0
        return {"progress": int(out[0]), "pending": int(out[1]), "evicted_state": int(out[2]), "bytes": int(out[3])}

    def reclaim_one_state(self, checkpoints_only, for_block): return bool(self.r.ref_cache_reclaim_one_state(self.h, int(checkpoints_only), for_block))

    def evict_all(self):
        out = (C.c_uint64 * 2)()
        assert self.r.ref_cache_evict_all(self.h, out) == 0
        return {"progress": bool(out[0]), "bytes": int(out[1])}

    def poll(self): self.r.ref_cache_poll(self.h)
    def complete(self, success=True): self.r.ref_cache_tier_complete(self.h, int(success))
    def tier_set(self, limit, writable=True): self.r.ref_cache_tier_set(self.h, limit, int(writable))

    def block_info(self, block):
        out = (C.c_uint64 * 8)()
        assert self.r.ref_cache_block_info(self.h, block, out) == 0
        if not out[0]:
            return None
        return {"page": int(out[1]), "transferring": bool(out[3]), "state": bool(out[5]), "state_resident": bool(out[6]),
                "state_ordinary": bool(out[7]), "poisoned": not out[4]}

    def snapshot(self):
        out = (C.c_uint64 * 16)()
        self.r.ref_cache_snapshot(self.h, out)
        names = ["pages_allocated", "pages_free", "pages_active", "pages_prefix", "states", "state_bytes", "pinned",
                 "tier_blocks", "pending_pages", "demotions", "restores", "demotions_refused", "kv_hit_tokens", "lazy_junctions",
                 "lost_state_misses", "probe_hashed_blocks"]
        return dict(zip(names, [int(x) for x in out]))


class Mine:
    def __init__(self, pages, extent, runway, budget, tier, slots, transfers):
        self.pool = KvPool(pages=pages, bytes_per_page=100, extent_pages=extent, runway_pages=runway, budget_pages=budget)
        self.cache = Cache(self.pool, Cache.MANUAL_TIER if tier else Cache.NO_TIER, slots, transfers)
        self.cache.set_state_coupled(True)
        if tier:
            self.cache.manual_tier_plain_limits(True)
        self.pinned = 0

    def close(self): self.cache.close(); self.pool.close()
    def begin(self, request): self.cache.begin_request(request)
    def end(self, request): self.cache.end_request(request)
    def ensure(self, request, tokens): return self.cache.ensure_tokens(request, tokens)
    def table(self, request): return self.cache.page_table(request)
    def publish(self, request, tokens, committed, images=None): self.cache.publish(request, tokens, committed, images)
    def block_at(self, request, boundary): return self.cache.block_at(request, boundary)

    def lookup(self, prompt, record=False, probe=None, images=None):
        found = self.cache.lookup_state(prompt, record=record, probe=probe, images=images)
        if found["state_block"]:
            self.cache.unpin_state(found["state_block"])
        blocks = found.pop("blocks")
        return found, blocks

    def attach(self, request, prompt, images=None):
        found = self.cache.lookup_state(prompt, images=images)
        blocks = found.pop("blocks")
        status = GRANTED
        if found["state_block"]:   # the chain up to its state; without a state nothing is restored
            status, _ = self.cache.attach_prefix(request, blocks[: found["resume_boundary"] // 32])
            self.cache.unpin_state(found["state_block"])
        return status, found

    def pin(self, prompt, images=None):
        found = self.cache.lookup_state(prompt, images=images)
        return found["state_block"]

    def unpin(self, block): self.cache.unpin_state(block)
    def probe(self, prompt, images=None): return self.cache.probe(prompt, images)
    def probe_refresh(self, handle, prompt, images=None): handle.refresh(prompt, images=images)
    def probe_tokens(self, handle): return handle.cached_tokens
    def probe_close(self, handle): handle.close()
    def restore_status(self, request): return self.cache.restore_status(request)
    def publish_state(self, block, size, checkpoint): self.cache.publish_state(block, size, checkpoint)
    def use(self, block, on): (self.cache.use_state if on else self.cache.unuse_state)(block)

    def publish_stored(self, block, size, checkpoint):
        self.cache.publish_stored_state(block, size, checkpoint)
        self.poll()

    def evict_one(self, up_to_in_use, keep_resume_point, pages_only):
        step = self.cache.evict_one(up_to_in_use, keep_resume_point, pages_only)
        return {k: step[k] for k in ("progress", "pending", "evicted_state")}

    def reclaim_step(self, mode, up_to_in_use, keep_resume_point, keep_runway):
        return self.cache.reclaim_step(mode, up_to_in_use, keep_resume_point, keep_runway)

    def reclaim_one_state(self, checkpoints_only, for_block): return self.cache.reclaim_one_state(checkpoints_only, for_block)
    def evict_all(self): return self.cache.evict_all()
    def poll(self): self.cache.poll_transfers()

    def complete(self, success=True):
        while self.cache.complete_transfer(success):
            pass

    def tier_set(self, limit, writable=True): self.cache.manual_tier_set(limit, writable)

    def block_info(self, block):
        found = self.cache.block_state(block)
        if found is None:
            return None
        state = self.cache.state_info(block)
        # (whether a block has a tier copy is compared through the tier's block count: there a copy counts from the start
        # of its write, here from its landing)
        return {"page": int(found["page"]), "transferring": found["transferring"], "state": bool(state["contains"]),
                "state_resident": bool(state["resident"]), "state_ordinary": bool(state["ordinary"]), "poisoned": found["poisoned"]}

    def snapshot(self):
        pool, cache, states, tier = self.pool.snapshot(), self.cache.snapshot(), self.cache.state_summary(), self.cache.tier_counters()
        return {"pages_allocated": int(pool["pages_allocated"]), "pages_free": int(pool["pages_free"]), "pages_active": int(pool["pages_active"]),
                "pages_prefix": int(pool["pages_prefix"]), "states": int(states["states"]), "state_bytes": int(states["bytes"]),
                "demotions": tier["demotions_landed"], "restores": tier["restores_landed"], "demotions_refused": tier["demotions_refused"],
                "pending_pages": tier["pending_pages"], "tier_blocks": int(cache["tier_blocks"]) + tier["pending_pages"],
                **self.cache.lookup_counters()}


def make_prompts(rng, count):
    """Prompts over a small alphabet of 32-token pages, so that chains share prefixes and branch."""
    pages = {letter: rng.integers(0, 50000, size=32, dtype=np.uint32) for letter in "abcd"}
    prompts = []
    for _ in range(count):
        if prompts and rng.random() < 0.6:   # branch off an earlier prompt
            base = prompts[rng.integers(len(prompts))][0]
            keep = int(rng.integers(0, len(base) + 1))
            letters = base[:keep] + "".join(rng.choice(list("abcd"), size=int(rng.integers(1, 4))))
        else:
            letters = "".join(rng.choice(list("abcd"), size=int(rng.integers(1, 6))))
        letters = letters[:6]
        tail = rng.integers(0, 50000, size=int(rng.integers(1, 32)), dtype=np.uint32)
        tokens = np.concatenate([pages[x] for x in letters] + [tail])
        # Some prompts carry images: token-identical pages then share a block only under the same image content. Two
        # digests over a few placements, so that both equal and differing identities occur.
        images = []
        if rng.random() < 0.4:
            at = 0
            while at + 8 < len(tokens) and len(images) < 3:
                at += int(rng.integers(0, 40))
                length = int(rng.choice([8, 16, 40]))
                if at + length > len(tokens):
                    break
                digest = int(rng.choice([0x1111, 0x3333]))
                images.append((at, length, 8, length // 4 if length >= 8 else 2, digest, digest + 1))
                at += length
        prompts.append((letters, tokens, images or None))
    return prompts


def run_trace(seed, steps, tier):
    rng = np.random.default_rng(seed)
    geometry = dict(pages=24, extent=int(rng.choice([1, 2, 4])), runway=0, budget=int(rng.choice([8, 12, 16])),
                    tier=tier, slots=int(rng.choice([2, 4, 16])), transfers=int(rng.choice([1, 2, 4])))
    geometry["budget"] -= geometry["budget"] % geometry["extent"]
    if tier:
        geometry["slots"] = 64   # a quota that never fills: replacement under a full quota involves the states' own tier
    mine, theirs = Mine(**geometry), Theirs(**geometry)
    prompts = make_prompts(rng, 10)
    active = {}      # request -> [prompt index, tokens ensured, tokens published]
    blocks = set()   # block ids seen
    used, pinned, probes = set(), [], []
    next_request = 1
    log = []

    def both(name, *args, **kwargs):
        a, b = getattr(mine, name)(*args, **kwargs), getattr(theirs, name)(*args, **kwargs)
        log.append((name, args, kwargs, a, b))
        return a, b

    def check(what):
        a, b = mine.snapshot(), theirs.snapshot()
        for key, value in a.items():
            assert value == b[key], (what, key, value, b[key], seed, log[-6:])
        for block in sorted(blocks):
            a, b = mine.block_info(block), theirs.block_info(block)
            assert a == b, (what, "block", block, a, b, seed, log[-6:])
        for request in active:
            assert mine.table(request) == theirs.table(request), (what, "page table", request, seed, log[-6:])
            assert mine.restore_status(request) == theirs.restore_status(request), (what, "restore status", request, seed, log[-6:])

    for step in range(steps):
        op = rng.choice(["begin", "grow", "publish", "end", "lookup", "state", "use", "evict", "poll", "pin", "reclaim", "state_reclaim", "probe", "tier", "evict_all"],
                        p=[0.10, 0.20, 0.18, 0.06, 0.05, 0.08, 0.04, 0.09, 0.07, 0.03, 0.04, 0.02, 0.03, 0.007, 0.003] if tier else
                          [0.10, 0.22, 0.20, 0.06, 0.06, 0.10, 0.05, 0.05, 0.02, 0.04, 0.04, 0.02, 0.037, 0.00, 0.003])
        if op == "begin" and len(active) < 4:
            request, next_request = next_request, next_request + 1
            index = int(rng.integers(len(prompts)))
            both("begin", request)
            active[request] = [index, 0, 0]
            if rng.random() < 0.7:   # resume from the cache
                (status_a, found_a), (status_b, found_b) = both("attach", request, prompts[index][1], images=prompts[index][2])
                assert status_a == status_b and found_a == found_b, ("attach", seed, status_a, status_b, found_a, found_b, log[-6:])
                if status_a == GRANTED:
                    active[request][1] = active[request][2] = len(mine.table(request)[0]) * 32
        elif op == "grow" and active:
            request = int(rng.choice(list(active)))
            index, ensured, published = active[request]
            target = min(len(prompts[index][1]), ensured + int(rng.integers(1, 80)))
            a, b = both("ensure", request, target)
            assert a == b, ("ensure", seed, a, b, log[-6:])
            if a == GRANTED:
                active[request][1] = max(ensured, target)
        elif op == "publish" and active:
            request = int(rng.choice(list(active)))
            index, ensured, published = active[request]
            if mine.restore_status(request) != 0:
                continue
            committed = int(rng.integers(published, ensured + 1)) if ensured > published else published
            both("publish", request, prompts[index][1], committed, images=prompts[index][2])
            active[request][2] = committed
            if committed >= 32 and rng.random() < 0.4:   # the engine publishes a state where the request stands
                block = mine.block_at(request, committed // 32 * 32)
                if mine.cache.block_state(block)["poisoned"]:
                    pass   # a request one of whose reads failed is ended, it publishes nothing more
                elif tier and rng.random() < 0.7 and not mine.cache.state_info(block)["contains"]:
                    both("publish_stored", block, 100, bool(rng.random() < 0.2))   # a state the model stores elsewhere
                else:
                    both("publish_state", block, 100, bool(rng.random() < 0.3))
            for boundary in range(32, committed + 1, 32):
                a, b = both("block_at", request, boundary)
                assert a == b, ("block_at", seed, a, b)
                blocks.add(a)
        elif op == "end" and active:
            request = int(rng.choice(list(active)))
            both("end", request)
            del active[request]
        elif op == "lookup":
            index = int(rng.integers(len(prompts)))
            record = bool(rng.random() < 0.5)
            (found_a, _), (found_b, _, _) = both("lookup", prompts[index][1], record=record, images=prompts[index][2])
            assert found_a == found_b, ("lookup", seed, found_a, found_b, log[-6:])
        elif op == "state" and blocks:
            block = int(rng.choice(sorted(blocks)))
            found = mine.cache.block_state(block)   # the engine publishes where a request stands: on a resident, readable block
            if found is None or found["page"] == 0xFFFFFFFF or found["transferring"] or found["poisoned"]:
                continue
            both("publish_state", block, int(rng.choice([100, 150, 200])), bool(rng.random() < 0.3))
        elif op == "use" and blocks:
            block = int(rng.choice(sorted(blocks)))
            if block in used:
                both("use", block, False)
                used.discard(block)
            elif mine.cache.block_state(block) is not None and mine.cache.state_info(block)["contains"]:
                both("use", block, True)
                used.add(block)
        elif op == "pin":
            if pinned and rng.random() < 0.6:
                block = pinned.pop(int(rng.integers(len(pinned))))
                both("unpin", block)
            else:
                index = int(rng.integers(len(prompts)))
                a, b = both("pin", prompts[index][1], images=prompts[index][2])
                assert a == b, ("pin", seed, a, b)
                if a:
                    pinned.append(a)
        elif op == "evict":
            args = (bool(rng.random() < 0.6), bool(rng.random() < 0.3), bool(rng.random() < 0.4))
            a, b = both("evict_one", *args)
            assert a == b, ("evict_one", seed, args, a, b, log[-6:])
        elif op == "reclaim":
            args = (int(rng.integers(0, 3)), bool(rng.random() < 0.6), bool(rng.random() < 0.3), bool(rng.random() < 0.3))
            a, b = both("reclaim_step", *args)
            assert a == b, ("reclaim_step", seed, args, a, b, log[-6:])
        elif op == "state_reclaim":
            args = (bool(rng.random() < 0.4), int(rng.choice(sorted(used))) if used and rng.random() < 0.5 else 0)
            a, b = both("reclaim_one_state", *args)
            assert a == b, ("reclaim_one_state", seed, args, a, b, log[-6:])
        elif op == "probe":   # what a scheduler keeps per waiting request between admission passes
            if len(probes) < 3 and rng.random() < 0.4:
                index = int(rng.integers(len(prompts)))
                probes.append((index, mine.probe(prompts[index][1], prompts[index][2]), theirs.probe(prompts[index][1], prompts[index][2])))
            elif probes:
                slot = int(rng.integers(len(probes)))
                index, a, b = probes[slot]
                choice = rng.random()
                if choice < 0.5:
                    mine.probe_refresh(a, prompts[index][1], prompts[index][2]); theirs.probe_refresh(b, prompts[index][1], prompts[index][2])
                elif choice < 0.8:   # an admission that acts on the probe, current or stale
                    (found_a, _), (found_b, _, _) = mine.lookup(prompts[index][1], record=True, probe=a, images=prompts[index][2]), theirs.lookup(prompts[index][1], record=True, probe=b, images=prompts[index][2])
                    assert found_a == found_b, ("probed lookup", seed, found_a, found_b, log[-6:])
                else:
                    mine.probe_close(a); theirs.probe_close(b)
                    probes.pop(slot)
                    slot = None
                if slot is not None:
                    assert mine.probe_tokens(a) == theirs.probe_tokens(b), ("probe", seed, mine.probe_tokens(a), theirs.probe_tokens(b), log[-6:])
            log.append(("probe", (), {}, None, None))
        elif op == "evict_all":   # a pressure pass: everything unpinned goes, then every extent that can be emptied
            a, b = both("evict_all")
            assert a == b, ("evict_all", seed, a, b, log[-6:])
        elif op == "tier":   # the tier takes fewer or more transfers at a time, or no writes at all (a failed write closed it)
            both("tier_set", int(rng.choice([0, 1, 2, 4])), bool(rng.random() < 0.8))
        elif op == "poll" and tier:
            if rng.random() < 0.7:
                both("complete", bool(rng.random() < 0.9))
            both("poll")
        else:
            continue
        check(op)
    for _, a, b in probes:
        mine.probe_close(a); theirs.probe_close(b)
    for block in pinned:
        both("unpin", block)
    for request in list(active):
        both("end", request)
    mine.complete(); theirs.complete()
    both("poll")
    mine.close(); theirs.close()


@pytest.mark.parametrize("seed", range(8))
def test_random_traces_without_a_tier_match_the_reference_facade(seed):
    run_trace(seed, 1500, tier=False)


@pytest.mark.parametrize("seed", range(8))
def test_random_traces_through_a_tier_match_the_reference_facade(seed):
    run_trace(100 + seed, 1500, tier=True)


def test_block_image_identity_equals_the_reference():
    """blockImageIdentity (runtime/engine/cache/KvCache.cpp:29-52) over random sorted spans and block positions, and
    the cases of the reference's own test (dev/tests/engine/kv_page_cache_test.cpp:35-84): text alone is zero, a block
    after the image carries nothing, the digest and the block's alignment inside the image both count, spans outside
    the block do not."""
    from richengine_b200 import lib as library
    mine = library.load()
    def identity_mine(begin, tokens, images):
        spans, n = image_spans(images)
        out = (C.c_uint64 * 2)()
        mine.rk_block_image_identity(begin, tokens, spans.ctypes.data if n else None, n, out)
        return int(out[0]), int(out[1])
    def identity_theirs(begin, tokens, images):
        spans, n = image_spans(images)
        out = (C.c_uint64 * 2)()
        reference.ref_block_image_identity(begin, tokens, spans.ctypes.data if n else None, n, out)
        return int(out[0]), int(out[1])
    red, blue, later, first = (8, 16, 8, 8, 0x1111, 0x2222), (8, 16, 8, 8, 0x3333, 0x4444), (40, 16, 8, 8, 0x1111, 0x2222), (0, 8, 4, 8, 0x5555, 0x6666)
    assert identity_mine(0, 32, None) == (0, 0) and identity_mine(32, 32, [red]) == (0, 0)
    assert identity_mine(0, 32, [red]) != (0, 0) and identity_mine(0, 32, [red]) != identity_mine(0, 32, [blue])
    assert identity_mine(32, 32, [later]) != identity_mine(0, 32, [red])
    assert identity_mine(32, 32, [first, blue, later]) == identity_mine(32, 32, [later]) and identity_mine(0, 8, [first, blue, later]) == identity_mine(0, 8, [first])
    rng = np.random.default_rng(9)
    for _ in range(300):
        spans, at = [], 0
        for _ in range(int(rng.integers(0, 5))):
            at += int(rng.integers(0, 50))
            length = int(rng.integers(1, 70))
            spans.append((at, length, int(rng.integers(1, 30)), int(rng.integers(1, 30)), int(rng.integers(0, 2 ** 63)), int(rng.integers(0, 2 ** 63))))
            at += length
        begin, tokens = int(rng.integers(0, 8)) * 32, int(rng.choice([8, 32]))
        assert identity_mine(begin, tokens, spans) == identity_theirs(begin, tokens, spans)
