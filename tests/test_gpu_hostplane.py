"""GPU: the host control plane over real device pages — prefix sharing with a copy-on-write fork,
then divergence; eviction of cold pages to pinned host memory and re-fetch on access; compaction
moves. Page bytes are compared with the CPU checker's mirror."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import dev, struct_to_device
from kvcase import HostPool, f32_to_bf16
from richengine_b200 import lib, ops
from richengine_b200.abi import INT4, INT8, Layout
from richengine_b200.hostplane import GRANTED, KV_BLOCK_LABEL_BYTES, NO_PAGE, Cache, KvPool, SlotStore
from richengine_b200.storage import PageStorage

pytestmark = pytest.mark.gpu


class World:
    """Device storage + pool + cache, with a host mirror of the same page ids for the checker."""

    def __init__(self, layout, pages, extent_pages, tier_slots=0):
        self.layout = layout
        self.storage = PageStorage(layout, pages, extent_pages)
        self.pool = KvPool(storage=self.storage, runway_pages=extent_pages)
        self.cache = Cache(self.pool, Cache.HOST_TIER if tier_slots else Cache.NO_TIER, tier_slots, 8)
        self.mirror = HostPool(layout, extent_pages, pages // extent_pages)
        self.rng = np.random.default_rng(0)

    def append(self, request, start, rows, mirror_too=True, seed=None):
        """Chunk-stores `rows` tokens at position `start` on the device (and on the host mirror)."""
        layout = self.layout
        rng = np.random.default_rng(seed if seed is not None else start * 7919 + rows)
        stride = (rows + 31) // 32 * 32
        k = f32_to_bf16(rng.standard_normal((4, stride, 256)).astype(np.float32))
        v = f32_to_bf16(rng.standard_normal((4, 256, stride)).astype(np.float32))
        pages, _, _ = self.cache.page_table(request)
        table = torch.zeros(len(pages), dtype=torch.int64, device="cuda")
        self.storage.write_entries(pages, 0, table)
        for layer in range(layout.attention_layers):
            place = self.storage.layers()[layer]
            ops.store_chunk(layout, dev(k), dev(v), table, lib.ChunkParams(start, rows, stride, len(pages), place))
            if mirror_too:
                host_table = self.mirror.table(pages)
                params = lib.ChunkParams(start, rows, stride, len(pages), self.mirror.layer(layer))
                assert om.oracle().rko_store_chunk(layout.format, 4, 256, k.ctypes.data, v.ctypes.data, host_table.ctypes.data, C.byref(params)) == 0
        torch.cuda.synchronize()

    def device_page(self, page):
        """The page's spans in layer, tensor order, from the device."""
        slot = torch.zeros(self.storage.bytes_per_page(), dtype=torch.uint8, device="cuda")
        ids = np.array([page], dtype=np.uint32)
        lib.check(lib.load().rk_storage_pack_pages(self.storage.handle, ids.ctypes.data, 1, slot.data_ptr(), 0, None), "pack")
        torch.cuda.synchronize()
        return slot.cpu().numpy()

    def mirror_page(self, page):
        return np.concatenate([self.mirror.tensor_view(page, layer, t) for layer in range(self.layout.attention_layers)
                               for t in range(4) if len(self.mirror.tensor_view(page, layer, t))])

    def close(self):
        self.cache.close(); self.pool.close(); self.storage.close()


def test_shared_prefix_fork_and_divergence():
    """Requests fork a published prefix, copy-on-write its partial tail page, then diverge; the shared
    pages stay bit-identical and every fork's own pages hold exactly what it appended."""
    layout = Layout(2, 4, 256, INT4)
    w = World(layout, 512, 128)
    prefix_tokens = 32 * 5 + 9  # five shared full pages and a partial tail
    ids = np.random.default_rng(1).integers(0, 1000, size=prefix_tokens + 100, dtype=np.uint32)
    w.cache.begin_request(1)
    assert w.cache.ensure_tokens(1, prefix_tokens) == GRANTED
    w.append(1, 0, prefix_tokens)
    w.cache.publish(1, ids, prefix_tokens)
    parent_pages = w.cache.page_table(1)[0]
    for child in (2, 3, 4):
        w.cache.begin_request(child)
        assert w.cache.fork(1, child, prefix_tokens) == 1
        pages = w.cache.page_table(child)[0]
        assert pages[:5] == parent_pages[:5] and pages[5] not in parent_pages
        torch.cuda.synchronize()
        assert np.array_equal(w.device_page(pages[5]), w.device_page(parent_pages[5]))  # the copy is exact
        # mirror the copy on the host, then let the child diverge by its own tokens
        om.oracle().rko_copy_page(INT4, 2, 4, 256, 128, w.mirror.entry(parent_pages[5]), w.mirror.entry(pages[5]))
        assert w.cache.ensure_tokens(child, prefix_tokens + 40) == GRANTED
        w.append(child, prefix_tokens, 40, seed=child)
    for request in (1, 2, 3, 4):
        for page in w.cache.page_table(request)[0]:
            assert np.array_equal(w.device_page(page), w.mirror_page(page)), (request, page)
    assert w.pool.snapshot()["pages_active"] == 6 + 3 * 2  # 6 parent pages; each child owns its tail copy + 1
    for request in (1, 2, 3, 4):
        w.cache.end_request(request)
    assert w.pool.snapshot()["pages_active"] == 0
    w.close()


def test_evict_cold_pages_to_pinned_host_and_refetch():
    """The coldest blocks go to pinned host memory (their pages return to the pool once the copy has
    landed); a later request that matches them gets fresh pages and the bytes come back exactly."""
    layout = Layout(2, 4, 256, INT8)
    w = World(layout, 256, 128, tier_slots=16)
    tokens = 32 * 8
    ids = np.random.default_rng(2).integers(0, 1000, size=tokens + 1, dtype=np.uint32)
    w.cache.begin_request(1)
    assert w.cache.ensure_tokens(1, tokens) == GRANTED
    w.append(1, 0, tokens)
    w.cache.publish(1, ids, tokens)
    pages = w.cache.page_table(1)[0]
    content = [w.device_page(p) for p in pages]
    for p, c in zip(pages, content):
        assert np.array_equal(c, w.mirror_page(p))
    w.cache.end_request(1)
    evicted = 0
    for _ in range(2):  # the coldest 25 %: two leaves, one after the other (a parent becomes a leaf next)
        assert w.cache.reclaim_one()
        while w.cache.snapshot()["transfers"]:
            w.cache.poll_transfers()
        evicted += 1
    snap = w.cache.snapshot()
    assert snap["tier_blocks"] == 2 and snap["resident_blocks"] == 6 and w.pool.snapshot()["pages_prefix"] == 6
    # scribble over the freed pages so a restore cannot pass by leftovers
    taken = w.pool.acquire(w.pool.snapshot()["pages_free"])
    junk = torch.full((w.storage.bytes_per_page(),), 0x5A, dtype=torch.uint8, device="cuda")
    for p in taken:
        ids32 = np.array([p], dtype=np.uint32)
        lib.check(lib.load().rk_storage_pack_pages(w.storage.handle, ids32.ctypes.data, 1, junk.data_ptr(), 1, None), "unpack")
    torch.cuda.synchronize()
    for p in reversed(taken):
        w.pool.release(p)
    chain = w.cache.lookup(ids)
    assert len(chain) == 8
    w.cache.begin_request(2)
    status, resume = w.cache.attach_prefix(2, chain)
    assert status == GRANTED and resume == tokens
    while w.cache.restores_pending(2):
        w.cache.poll_transfers()
    restored = w.cache.page_table(2)[0]
    assert restored[:6] == pages[:6]
    for i, p in enumerate(restored):
        assert np.array_equal(w.device_page(p), content[i]), i
    # a failed demotion loses nothing: the page stays resident and matchable
    w.cache.end_request(2)
    assert w.cache.reclaim_one() and w.cache.reclaim_one()  # both leaves still have their host copies: dropped at once
    assert w.cache.snapshot()["transfers"] == 0 and w.pool.snapshot()["pages_prefix"] == 6
    w.cache.fail_next_transfers(1)
    assert w.cache.reclaim_one()                             # the next leaf has no copy yet: a demotion, which fails
    while w.cache.snapshot()["transfers"]:
        w.cache.poll_transfers()
    assert w.cache.snapshot()["failed_transfers"] == 1 and w.pool.snapshot()["pages_prefix"] == 6
    assert len(w.cache.lookup(ids)) == 8
    w.close()


def test_kv_survives_a_restart_through_the_slot_store(tmp_path):
    """Every block goes to the pinned-host tier (its CRC-32C taken on the GPU when it is packed), the cache seals the
    tier into a slot file, everything is torn down; new storage, pool, tier and cache adopt the file, a request matching
    the prompt gets the bytes back exactly, and a payload changed on disk fails its first restore: a miss."""
    layout = Layout(2, 4, 256, INT4)
    tokens = 32 * 6
    ids = np.random.default_rng(7).integers(0, 1000, size=tokens + 1, dtype=np.uint32)
    w = World(layout, 256, 128, tier_slots=16)
    w.cache.begin_request(1)
    assert w.cache.ensure_tokens(1, tokens) == GRANTED
    w.append(1, 0, tokens, mirror_too=False)
    w.cache.publish(1, ids, tokens)
    content = [w.device_page(p) for p in w.cache.page_table(1)[0]]
    w.cache.end_request(1)
    while w.cache.reclaim_one():
        while w.cache.snapshot()["transfers"]:
            w.cache.poll_transfers()
    assert w.cache.snapshot()["tier_blocks"] == 6 and w.cache.snapshot()["resident_blocks"] == 0
    slot_bytes = (w.storage.bytes_per_page() + 4095) // 4096 * 4096
    files = dict(slots_path=tmp_path / "kv.slots", records_path=tmp_path / "kv.records", tag=b"int4 2x4x256",
                 label_bytes=KV_BLOCK_LABEL_BYTES, slot_bytes=slot_bytes)
    store = SlotStore(**files)
    assert w.cache.persist(store) == 6
    store.close()
    w.close()

    # the record's checksum is the device's CRC-32C of the packed page: the checker agrees on the file's bytes
    store = SlotStore(**files)
    records = store.records()
    assert len(records) == 6
    for record, page in zip(records, content):
        payload = store.read(record["index"], record["payload_bytes"])
        assert record["payload_bytes"] == len(page) and np.array_equal(payload, page)
        assert record["checksum"] == om.oracle().rko_crc32c(payload.ctypes.data, len(payload), 0)
    store.close()
    with open(tmp_path / "kv.slots", "r+b") as f:  # one bit of the fifth block's payload changes on disk
        f.seek(records[4]["index"] * slot_bytes + 12345)
        byte = f.read(1)
        f.seek(records[4]["index"] * slot_bytes + 12345)
        f.write(bytes([byte[0] ^ 1]))

    w = World(layout, 256, 128, tier_slots=16)
    store = SlotStore(**files)
    assert w.cache.adopt(store) == {"blocks": 6, "dropped": 0, "bytes": 6 * w.storage.bytes_per_page()}
    chain = w.cache.lookup(ids)
    assert len(chain) == 6
    w.cache.begin_request(2)
    status, resume = w.cache.attach_prefix(2, chain)
    assert status == GRANTED and resume == tokens
    while w.cache.restores_pending(2):
        w.cache.poll_transfers()
    assert w.cache.snapshot()["failed_transfers"] == 1  # the changed payload did not match its record
    restored = w.cache.page_table(2)[0]
    for i in range(4):
        assert np.array_equal(w.device_page(restored[i]), content[i]), i
    assert len(w.cache.lookup(ids)) == 4                 # the chain ends before the damaged block
    w.cache.end_request(2)
    store.close()
    w.close()


def test_restore_points_survive_a_restart_with_their_chains(tmp_path):
    """State-coupled, as the reference's hybrid model runs: two stored composite states (after three and after six
    pages) are the restore points. Everything goes to the pinned-host tier and into the slot file, the state labels are
    written as a clean stop writes them; the next process takes both points back with their chains, a request resumes
    at the deeper state and gets the device bytes back exactly."""
    layout = Layout(2, 4, 256, INT4)
    tokens = 32 * 6
    ids = np.random.default_rng(9).integers(0, 1000, size=tokens + 1, dtype=np.uint32)
    w = World(layout, 256, 128, tier_slots=16)
    w.cache.set_state_coupled(True)
    w.cache.begin_request(1)
    assert w.cache.ensure_tokens(1, tokens) == GRANTED
    w.append(1, 0, tokens, mirror_too=False)
    w.cache.publish(1, ids, tokens)
    content = [w.device_page(p) for p in w.cache.page_table(1)[0]]
    w.cache.publish_stored_state(w.cache.block_at(1, 96), 4096)
    w.cache.publish_stored_state(w.cache.block_at(1, tokens), 4096, checkpoint=True)
    w.cache.poll_transfers()
    w.cache.end_request(1)
    for _ in range(64):
        w.cache.evict_all()
        while w.cache.snapshot()["transfers"]:
            w.cache.poll_transfers()
        if w.cache.snapshot()["resident_blocks"] == 0:
            break
    assert w.cache.snapshot()["tier_blocks"] == 6 and w.cache.snapshot()["resident_blocks"] == 0
    slot_bytes = (w.storage.bytes_per_page() + 4095) // 4096 * 4096
    files = dict(slots_path=tmp_path / "kv.slots", records_path=tmp_path / "kv.records", tag=b"int4 2x4x256",
                 label_bytes=KV_BLOCK_LABEL_BYTES, slot_bytes=slot_bytes)
    store = SlotStore(**files)
    assert w.cache.persist(store) == 6
    points = w.cache.state_labels()
    assert [(np.frombuffer(label, "<u4", offset=16)[0], size) for label, size in points] == [(96, 4096), (tokens, 4096)]
    store.close()
    w.close()

    w = World(layout, 256, 128, tier_slots=16)
    w.cache.set_state_coupled(True)
    store = SlotStore(**files)
    assert w.cache.adopt_restore_points(store, points) == {"blocks": 6, "dropped": 0, "bytes": 6 * w.storage.bytes_per_page() + 2 * 4096, "states": 2}
    found = w.cache.lookup_state(ids)
    assert found["kv_boundary"] == found["resume_boundary"] == tokens and len(found["blocks"]) == 6
    w.cache.begin_request(2)
    status, resume = w.cache.attach_prefix(2, found["blocks"])
    assert status == GRANTED and resume == tokens
    while w.cache.restores_pending(2):
        w.cache.poll_transfers()
    assert w.cache.snapshot()["failed_transfers"] == 0
    for page, want in zip(w.cache.page_table(2)[0], content):
        assert np.array_equal(w.device_page(page), want)
    if found["state_block"]:
        w.cache.unpin_state(found["state_block"])
    w.cache.end_request(2)
    store.close()
    w.close()


def test_pool_compaction_moves_device_pages():
    layout = Layout(1, 4, 256, INT4)
    w = World(layout, 384, 128)
    w.cache.begin_request(1)
    assert w.cache.ensure_tokens(1, 32 * 200) == GRANTED  # spills into a second extent
    w.append(1, 0, 32 * 6)
    before = w.cache.page_table(1)[0]
    kept = [w.device_page(p) for p in before[:6]]
    assert w.cache.truncate(1, 32 * 6, 0) == 194
    w.cache.begin_request(2)
    assert w.cache.ensure_tokens(2, 32 * 130) == GRANTED
    w.cache.end_request(2)
    if w.cache.compact_extent():
        torch.cuda.synchronize()
    after = w.cache.page_table(1)[0]
    for i, p in enumerate(after):
        assert np.array_equal(w.device_page(p), kept[i])
    w.cache.end_request(1)
    w.close()
