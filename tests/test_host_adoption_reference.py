"""CPU: taking back sealed tier copies, side by side with the reference's OWN Cache::adopt
(runtime/engine/cache/Cache.cpp:38-141 compiled in place into oracle/_ref, over the reference's persistent test tier,
dev/tests/engine/TestKvTier.hpp). Both read the same KvBlockLabel bytes (runtime/engine/cache/DiskLabels.hpp:22-29):
this repository's cache from the records of a slot store, the reference's from the label list a persistent tier hands
it. The reference takes a chain back only for a composite state; here every record gets a stored state at its depth in
the label forest, so that every whole chain is wanted and the two decisions can be compared record by record: ids in
id order, first record of an id wins, a parent at or above its child, a missing link, a key another block already
holds, and where new ids continue."""
import ctypes as C

import numpy as np
import pytest

import oracle as om
from richengine_b200 import lib
from richengine_b200.hostplane import GRANTED, KV_BLOCK_LABEL_BYTES, STATE_LABEL_BYTES, Cache, KvPool, SlotStore, kv_block_label, state_label

reference = om.reference()
pytestmark = pytest.mark.skipif(reference is None or not hasattr(reference, "ref_cache_adopt"),
                                reason="the reference's cache facade was not compiled here")

SLOT = 100  # the reference's test tier has 100-byte slots


def crc(payload):
    return lib.load().rk_crc32c_host(payload.ctypes.data, payload.size, 0)


def mine_fresh(pages=64):
    pool = KvPool(pages=pages, bytes_per_page=SLOT, extent_pages=8, runway_pages=0, budget_pages=pages)
    return pool, Cache(pool, Cache.MANUAL_TIER, 256, 8)


def theirs_fresh(pages=64):
    handle = reference.ref_cache_create(pages, SLOT, 8, 0, pages, 2, 256, 8)  # 2: a persistent tier
    assert handle
    return handle


def write_labels(tmp_path, labels, name="a"):
    """One slot per label at ascending indices, payload = the slot number repeated, then "the next process" opens it."""
    paths = (tmp_path / f"{name}.slots", tmp_path / f"{name}.records")
    store = SlotStore(*paths, b"adoption", KV_BLOCK_LABEL_BYTES, 4096)
    for index, label in enumerate(labels):
        payload = np.full(SLOT, index % 251, np.uint8)
        assert store.write(index, payload, crc(payload), label)
    assert store.synchronize()
    store.close()
    return SlotStore(*paths, b"adoption", KV_BLOCK_LABEL_BYTES, 4096)


def fields(label):
    head = np.frombuffer(label, dtype="<u8", count=5)
    return {"id": int(head[0]), "parent": int(head[1]), "last_used": int(head[2]), "images": (int(head[3]), int(head[4])),
            "tokens": np.frombuffer(label, dtype="<u4", offset=40)}


def depths(labels):
    """Tokens up to and including each id in the label forest (first record of an id counts; 0 = no whole chain)."""
    first = {}
    for label in labels:
        f = fields(label)
        if f["id"] and f["parent"] < f["id"]:
            first.setdefault(f["id"], f)
    depth = {}
    for block in sorted(first):
        parent = first[block]["parent"]
        depth[block] = 32 if not parent else (depth.get(parent, 0) + 32 if depth.get(parent, 0) else 0)
    return depth


def reference_adopt(handle, labels, states):
    blob = np.frombuffer(b"".join(labels), np.uint8) if labels else np.zeros(1, np.uint8)
    sizes = np.array([len(label) for label in labels] or [0], np.uint32)
    blocks = np.array([s[0] for s in states] or [0], np.uint64)
    tokens = np.array([s[1] for s in states] or [0], np.uint32)
    used = np.array([s[2] for s in states] or [0], np.uint64)
    out = (C.c_uint64 * 4)()
    status = reference.ref_cache_adopt(handle, blob.ctypes.data, sizes.ctypes.data, len(labels), blocks.ctypes.data,
                                       tokens.ctypes.data, used.ctypes.data, len(states), out)
    assert status == 0
    return {"states": int(out[0]), "blocks": int(out[1]), "bytes": int(out[2]), "dropped": int(out[3])}


def reference_has(handle, block):
    info = (C.c_uint64 * 8)()
    assert reference.ref_cache_block_info(handle, block, info) == 0
    return bool(info[0])


def random_forest(rng, count, vocabulary=6):
    """Labels of a forest with the defects a damaged or stale record set can show. A small vocabulary of token pages
    makes key collisions (same parent, same 32 tokens, another id) frequent."""
    pages = [rng.integers(0, 50000, size=32, dtype=np.uint32) for _ in range(vocabulary)]
    labels, ids = [], []
    next_id = 1
    for _ in range(count):
        next_id += int(rng.integers(0, 3))          # gaps: ids the earlier process gave to blocks it dropped again
        block = next_id
        next_id += 1
        parent = 0 if not ids or rng.random() < 0.25 else int(rng.choice(ids))
        roll = rng.random()
        if roll < 0.04:
            parent = block + int(rng.integers(0, 3))  # a parent at or above its child
        elif roll < 0.08:
            parent = next_id + 50 if rng.random() < 0.5 else max(1, block - 1)  # a link to nothing, or to whatever sits there
        elif roll < 0.11:
            block = 0
        elif roll < 0.16 and ids:
            block = int(rng.choice(ids))              # a second record of an id: a stale one
        images = (0, 0) if rng.random() < 0.8 else (int(rng.integers(1, 1 << 62)), int(rng.integers(1, 1 << 62)))
        labels.append(kv_block_label(block, parent, int(rng.integers(1, 10_000)), pages[int(rng.integers(0, vocabulary))], images))
        if block:
            ids.append(block)
    order = rng.permutation(len(labels))              # slots are reused: file order says nothing about age
    return [labels[i] for i in order]


@pytest.mark.parametrize("seed", range(60))
def test_adoption_of_a_damaged_record_set_equals_the_reference(tmp_path, seed):
    rng = np.random.default_rng(seed)
    labels = random_forest(rng, int(rng.integers(1, 40)))
    store = write_labels(tmp_path, labels)
    recorded = [r["label"] for r in store.records()]
    assert sorted(recorded) == sorted(labels)
    pool, cache = mine_fresh()
    mine = cache.adopt(store)

    depth = depths(recorded)
    states = [(block, tokens, 1) for block, tokens in depth.items() if tokens]
    handle = theirs_fresh()
    theirs = reference_adopt(handle, recorded, states)
    try:
        every = {fields(label)["id"] for label in recorded} | {0}
        kept_mine = {block for block in every if block and cache.block_state(block) is not None}
        kept_theirs = {block for block in every if block and reference_has(handle, block)}
        assert kept_mine == kept_theirs, f"seed {seed}: mine only {sorted(kept_mine - kept_theirs)}, reference only {sorted(kept_theirs - kept_mine)}"
        assert mine["blocks"] == theirs["blocks"] == len(kept_mine)
        assert mine["bytes"] == mine["blocks"] * SLOT
        # the reference's count also holds the states it left behind
        assert mine["dropped"] == theirs["dropped"] - (len(states) - theirs["states"]), (mine, theirs, len(states))
        # a block published now gets the same id in both: after every id a record named, taken back or not
        fresh = np.arange(900_000, 900_033, dtype=np.uint32)
        cache.begin_request(1)
        assert cache.ensure_tokens(1, 32) == GRANTED
        cache.publish(1, fresh, 32)
        assert reference.ref_cache_begin(handle, 1) == 0
        assert reference.ref_cache_ensure(handle, 1, 32) == 0
        assert reference.ref_cache_publish(handle, 1, fresh.ctypes.data, len(fresh), 32, None, 0) == 0
        assert cache.block_at(1, 32) == reference.ref_cache_block_at(handle, 1, 32) > max(every)
    finally:
        reference.ref_cache_destroy(handle)
        store.close(); cache.close(); pool.close()


def random_states(rng, recorded):
    """Stored states over a label forest: at some blocks with whole chains, plus the defects of a stale state file — a
    boundary that is not the chain's length, a block no record names, a block whose chain is broken, a second state of
    one block. (block, last used, tokens, checkpoint), the order of a StateLabel's fields."""
    depth = depths(recorded)
    states = []
    for block, tokens in depth.items():
        roll = rng.random()
        if roll < 0.35:
            states.append((block, int(rng.integers(1, 20_000)), tokens or 32, bool(rng.random() < 0.3)))  # a broken chain's state claims one page
        elif roll < 0.40:
            states.append((block, int(rng.integers(1, 20_000)), tokens + 32, False))
        if roll < 0.05:
            states.append((block, int(rng.integers(1, 20_000)), tokens or 32, bool(rng.random() < 0.5)))
    if rng.random() < 0.5:
        states.append((max(depth, default=0) + int(rng.integers(1, 40)), 7, 32, False))
    return [states[i] for i in rng.permutation(len(states))]


def reference_adopt_points(handle, labels, states):
    blob = np.frombuffer(b"".join(labels), np.uint8) if labels else np.zeros(1, np.uint8)
    sizes = np.array([len(label) for label in labels] or [0], np.uint32)
    packed = b"".join(state_label(*state) for state in states)
    out = (C.c_uint64 * 4)()
    assert reference.ref_cache_adopt_labelled(handle, blob.ctypes.data, sizes.ctypes.data, len(labels), packed, len(states), out) == 0
    return {"states": int(out[0]), "blocks": int(out[1]), "bytes": int(out[2]), "dropped": int(out[3])}


@pytest.mark.parametrize("seed", range(60))
def test_adoption_of_restore_points_equals_the_reference(tmp_path, seed):
    """The reference's own rule (Cache.cpp:70-127): a state comes back with its whole chain, a block only for a state.
    The same block labels and the same state labels on both sides: blocks and states taken back, everything left
    behind, the bytes held, the next block id, and the labels a clean stop writes for the states afterwards."""
    rng = np.random.default_rng(1000 + seed)
    labels = random_forest(rng, int(rng.integers(1, 40)))
    store = write_labels(tmp_path, labels)
    recorded = [r["label"] for r in store.records()]
    states = random_states(rng, recorded)
    pool, cache = mine_fresh()
    cache.set_state_coupled(True)
    mine = cache.adopt_restore_points(store, [(state_label(*state), 64) for state in states])
    handle = theirs_fresh()
    theirs = reference_adopt_points(handle, recorded, states)
    try:
        every = {fields(label)["id"] for label in recorded} | {state[0] for state in states} | {0}
        kept_mine = {block for block in every if block and cache.block_state(block) is not None}
        kept_theirs = {block for block in every if block and reference_has(handle, block)}
        assert kept_mine == kept_theirs, f"seed {seed}: mine only {sorted(kept_mine - kept_theirs)}, reference only {sorted(kept_theirs - kept_mine)}"
        assert mine == theirs, (mine, theirs)
        blob, sizes = np.zeros(256 * STATE_LABEL_BYTES, np.uint8), np.zeros(256, np.uint64)
        count = reference.ref_cache_state_labels(handle, blob.ctypes.data, sizes.ctypes.data, 256)
        assert count == theirs["states"]
        written = sorted((blob[i * STATE_LABEL_BYTES:(i + 1) * STATE_LABEL_BYTES].tobytes(), int(sizes[i])) for i in range(count))
        assert sorted(cache.state_labels()) == written
        fresh = np.arange(900_000, 900_033, dtype=np.uint32)
        cache.begin_request(1)
        assert cache.ensure_tokens(1, 32) == GRANTED
        cache.publish(1, fresh, 32)
        assert reference.ref_cache_begin(handle, 1) == 0
        assert reference.ref_cache_ensure(handle, 1, 32) == 0
        assert reference.ref_cache_publish(handle, 1, fresh.ctypes.data, len(fresh), 32, None, 0) == 0
        assert cache.block_at(1, 32) == reference.ref_cache_block_at(handle, 1, 32) > max(every)
    finally:
        reference.ref_cache_destroy(handle)
        store.close(); cache.close(); pool.close()


def reference_seals(prompts):
    """The reference, persistent: publishes each prompt's full pages, evicts everything to its tier and hands over the
    labels its slots carry (Cache::labelKv, Cache.cpp:853-860)."""
    handle = theirs_fresh()
    for request, prompt in enumerate(prompts, start=1):
        full = len(prompt) // 32 * 32
        assert reference.ref_cache_begin(handle, request) == 0
        assert reference.ref_cache_ensure(handle, request, full) == 0
        assert reference.ref_cache_publish(handle, request, prompt.ctypes.data, len(prompt), full, None, 0) == 0
        # a persistent cache keeps a chain on its tier only for a restore point: a stored state at the chain's end
        assert reference.ref_cache_publish_state_stored(handle, reference.ref_cache_block_at(handle, request, full), 64, 0) == 0
        assert reference.ref_cache_poll(handle) >= 0
        assert reference.ref_cache_end(handle, request) == 0
    out = (C.c_uint64 * 4)()
    for _ in range(200):
        assert reference.ref_cache_evict_one(handle, 1, 0, 0, out) == 0
        reference.ref_cache_tier_complete(handle, 1)
        assert reference.ref_cache_poll(handle) >= 0
        if not out[0] and not out[1]:
            break
    snapshot = (C.c_uint64 * 16)()
    reference.ref_cache_snapshot(handle, snapshot)
    blob = np.zeros(256 * KV_BLOCK_LABEL_BYTES, np.uint8)
    count = reference.ref_cache_tier_labels(handle, blob.ctypes.data, 256)
    assert count == snapshot[7] > 0, "every copy on the tier carries a label"
    labels = [blob[i * KV_BLOCK_LABEL_BYTES:(i + 1) * KV_BLOCK_LABEL_BYTES].tobytes() for i in range(count)]
    return handle, sorted(labels, key=lambda label: fields(label)["id"])


def reference_state_labels(handle):
    blob, sizes = np.zeros(256 * STATE_LABEL_BYTES, np.uint8), np.zeros(256, np.uint64)
    count = reference.ref_cache_state_labels(handle, blob.ctypes.data, sizes.ctypes.data, 256)
    assert count >= 0
    return sorted((blob[i * STATE_LABEL_BYTES:(i + 1) * STATE_LABEL_BYTES].tobytes(), int(sizes[i])) for i in range(count))


def prompts_for(seed):
    rng = np.random.default_rng(seed)
    base = rng.integers(0, 50000, size=161, dtype=np.uint32)
    branch = np.concatenate([base[:64], rng.integers(0, 50000, size=70, dtype=np.uint32)])
    other = rng.integers(0, 50000, size=97, dtype=np.uint32)
    return [base, branch, other]


def test_labels_the_reference_wrote_are_taken_back_here_and_sealed_again_byte_for_byte(tmp_path):
    prompts = prompts_for(3)
    handle, labels = reference_seals(prompts)
    points = reference_state_labels(handle)   # what its clean stop writes for the three restore points
    reference.ref_cache_destroy(handle)
    assert len(labels) == 5 + 2 + 3 and len(points) == 3
    store = write_labels(tmp_path, labels)
    pool, cache = mine_fresh()
    assert cache.adopt(store) == {"blocks": len(labels), "dropped": 0, "bytes": len(labels) * SLOT}
    # sealed again by this cache before anything touched a block's recency, the records name the same blocks with the same bytes
    again = SlotStore(tmp_path / "b.slots", tmp_path / "b.records", b"adoption", KV_BLOCK_LABEL_BYTES, 4096)
    assert cache.persist(again) == len(labels)
    again.close()
    again = SlotStore(tmp_path / "b.slots", tmp_path / "b.records", b"adoption", KV_BLOCK_LABEL_BYTES, 4096)
    assert sorted(r["label"] for r in again.records()) == sorted(labels)
    again.close()
    for prompt in prompts:
        assert len(cache.lookup(np.concatenate([prompt, [1]]))) == len(prompt) // 32
    store.close(); cache.close(); pool.close()
    # with the state labels, under the reference's rule: the three restore points and their chains, and a clean stop
    # here writes the state labels the reference wrote
    store = write_labels(tmp_path, labels, name="c")
    pool, cache = mine_fresh()
    cache.set_state_coupled(True)
    assert cache.adopt_restore_points(store, points) == {"blocks": len(labels), "dropped": 0, "bytes": len(labels) * SLOT + 3 * 64, "states": 3}
    assert sorted(cache.state_labels()) == points
    for prompt in prompts:
        found = cache.lookup_state(np.concatenate([prompt, [1]]))
        assert found["kv_boundary"] == found["resume_boundary"] == len(prompt) // 32 * 32
    store.close(); cache.close(); pool.close()


def test_labels_sealed_here_equal_the_reference_s_own_for_the_same_history(tmp_path):
    """The same requests on both sides, everything evicted: this cache's seal names each block as the reference's tier
    labels do — id, parent, image identity and tokens; the recency stamp is each side's clock at its own eviction."""
    prompts = prompts_for(11)
    handle, theirs = reference_seals(prompts)
    pool, cache = mine_fresh()
    for request, prompt in enumerate(prompts, start=1):
        full = len(prompt) // 32 * 32
        cache.begin_request(request)
        assert cache.ensure_tokens(request, full) == GRANTED
        cache.publish(request, prompt, full)
        cache.end_request(request)
    while cache.reclaim_one():
        assert cache.complete_transfer(True)
        cache.poll_transfers()
    store = SlotStore(tmp_path / "m.slots", tmp_path / "m.records", b"adoption", KV_BLOCK_LABEL_BYTES, 4096)
    assert cache.persist(store) == len(theirs)
    store.close()
    store = SlotStore(tmp_path / "m.slots", tmp_path / "m.records", b"adoption", KV_BLOCK_LABEL_BYTES, 4096)
    mine = sorted((r["label"] for r in store.records()), key=lambda label: fields(label)["id"])
    for a, b in zip(mine, theirs):
        fa, fb = fields(a), fields(b)
        assert (fa["id"], fa["parent"], fa["images"]) == (fb["id"], fb["parent"], fb["images"]) and (fa["tokens"] == fb["tokens"]).all()
    # and the reference takes this cache's seal back whole
    reference.ref_cache_destroy(handle)
    handle = theirs_fresh()
    depth = depths(mine)
    result = reference_adopt(handle, mine, [(block, tokens, fields(label)["last_used"]) for label in mine
                                            for block, tokens in [(fields(label)["id"], depth[fields(label)["id"]])]])
    assert result["blocks"] == len(mine) and result["dropped"] == 0 and result["states"] == len(mine)
    reference.ref_cache_destroy(handle)
    store.close(); cache.close(); pool.close()


def test_the_random_restore_point_sets_take_states_and_chains_back(tmp_path):
    """The comparison above is not one of two empty caches: over its seeds hundreds of states and chains come back and
    about as many records and states stay behind."""
    taken = {"blocks": 0, "states": 0, "dropped": 0}
    for seed in range(60):
        rng = np.random.default_rng(1000 + seed)
        labels = random_forest(rng, int(rng.integers(1, 40)))
        folder = tmp_path / str(seed)
        folder.mkdir()
        store = write_labels(folder, labels)
        states = random_states(rng, [r["label"] for r in store.records()])
        pool, cache = mine_fresh()
        result = cache.adopt_restore_points(store, [(state_label(*state), 64) for state in states])
        for key in taken:
            taken[key] += result[key]
        store.close(); cache.close(); pool.close()
    assert taken["states"] > 200 and taken["blocks"] > 300 and taken["dropped"] > 500, taken


def test_restore_points_come_back_only_into_an_empty_cache(tmp_path):
    """Cache::adopt refuses once anything is in the cache (Cache.cpp:41-42); a state without bytes is no stored copy and
    stays behind with the chain only it wanted."""
    tokens = np.arange(32, dtype=np.uint32)
    labels = [kv_block_label(1, 0, 5, tokens), kv_block_label(2, 1, 6, tokens + 100)]
    store = write_labels(tmp_path, labels)
    pool, cache = mine_fresh()
    cache.begin_request(1)
    with pytest.raises(RuntimeError):
        cache.adopt_restore_points(store, [(state_label(1, 5, 32), 64)])
    cache.end_request(1)
    assert cache.adopt_restore_points(store, [(state_label(1, 5, 32), 64), (state_label(2, 6, 64), 0)]) == \
        {"blocks": 1, "dropped": 2, "bytes": SLOT + 64, "states": 1}
    assert cache.block_state(1) is not None and cache.block_state(2) is None
    with pytest.raises(RuntimeError):
        cache.adopt_restore_points(store, [])
    store.close(); cache.close(); pool.close()
