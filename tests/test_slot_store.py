"""CPU: the persistent slot store — record and header bytes against a restatement of the reference's format
(runtime/model/SlotFile.cpp:238-323), reopening rules (:398-438), and a cache that seals its tier copies and takes
them back in a new process's objects (runtime/engine/cache/Cache.cpp:38-140)."""
import struct

import numpy as np
import pytest

import oracle as om
from richengine_b200 import lib
from richengine_b200.hostplane import (GRANTED, KV_BLOCK_LABEL_BYTES, NO_PAGE, Cache, KvPool, SlotStore, kv_block_label)


def crc(data: bytes) -> int:
    buffer = np.frombuffer(data, dtype=np.uint8)
    return om.oracle().rko_crc32c(buffer.ctypes.data if data else None, len(data), 0)


def expected_header(slot_bytes, label_bytes, tag: bytes) -> bytes:
    """{magic[8], version, label bytes, slot bytes (u64), tag bytes, checksum} + tag; the checksum covers both with a zero field."""
    blank = b"SPLASHSF" + struct.pack("<IIQII", 1, label_bytes, slot_bytes, len(tag), 0) + tag
    return b"SPLASHSF" + struct.pack("<IIQII", 1, label_bytes, slot_bytes, len(tag), crc(blank)) + tag


def expected_record(label_bytes, payload_bytes, checksum, label: bytes) -> bytes:
    """{0x53524543, payload checksum, payload bytes (u64)} + label + CRC-32C of all that, zero-padded to 64 bytes."""
    covered = struct.pack("<IIQ", 0x53524543, checksum, payload_bytes) + label
    size = (16 + label_bytes + 4 + 63) // 64 * 64
    return (covered + struct.pack("<I", crc(covered))).ljust(size, b"\0")


def test_record_and_header_bytes():
    library = lib.load()
    assert library.rk_slot_record_bytes(168) == 192 and library.rk_slot_record_bytes(24) == 64 and library.rk_slot_record_bytes(44) == 64
    assert library.rk_slot_record_bytes(45) == 128
    label = kv_block_label(7, 3, 99, list(range(100, 132)), images=(5, 6))
    assert len(label) == KV_BLOCK_LABEL_BYTES
    out = np.zeros(192, np.uint8)
    assert library.rk_slot_record_encode(168, 540672, 0xDEADBEEF, label, out.ctypes.data) == lib.OK
    assert out.tobytes() == expected_record(168, 540672, 0xDEADBEEF, label)
    tag = b"int4/16x4x256"
    header = np.zeros(4096, np.uint8)
    size = library.rk_slot_records_header(540672, 168, tag, len(tag), header.ctypes.data, 4096)
    assert size == 32 + len(tag) and header[:size].tobytes() == expected_header(540672, 168, tag)
    assert library.rk_slot_records_header(4096, 8, bytes(4096), 4096, header.ctypes.data, 4096) == lib.INVALID  # tag too long


def open_store(tmp_path, tag=b"tag-a", label_bytes=24, slot_bytes=8192):
    return SlotStore(tmp_path / "slots", tmp_path / "records", tag, label_bytes, slot_bytes)


def test_files_hold_the_reference_format_and_reopen(tmp_path):
    rng = np.random.default_rng(1)
    store = open_store(tmp_path)
    assert store.records() == []
    payloads = {0: rng.integers(0, 256, 8192, dtype=np.uint8), 2: rng.integers(0, 256, 5000, dtype=np.uint8)}
    labels = {0: bytes(range(24)), 2: bytes(range(50, 74))}
    for index, payload in payloads.items():
        assert store.write(index, payload, crc(payload.tobytes()), labels[index])
    assert store.synchronize()
    store.close()
    records = (tmp_path / "records").read_bytes()
    assert records[:37] == expected_header(8192, 24, b"tag-a") and records[37:4096] == bytes(4096 - 37)
    assert len(records) == 4096 + 3 * 64
    assert records[4096:4160] == expected_record(24, 8192, crc(payloads[0].tobytes()), labels[0])
    assert records[4160:4224] == bytes(64)  # index 1 was never written: a free slot
    assert records[4224:4288] == expected_record(24, 5000, crc(payloads[2].tobytes()), labels[2])
    slots = (tmp_path / "slots").read_bytes()
    assert slots[:8192] == payloads[0].tobytes() and slots[16384:16384 + 5000] == payloads[2].tobytes()
    assert slots[16384 + 5000:] == bytes(8192 - 5000)  # a write zeros the rest of its slot
    again = open_store(tmp_path)
    found = again.records()
    assert [(r["index"], r["payload_bytes"], r["checksum"], r["label"]) for r in found] == \
        [(i, payloads[i].size, crc(payloads[i].tobytes()), labels[i]) for i in (0, 2)]
    assert (again.read(2, 5000) == payloads[2]).all()
    assert again.free(0)
    again.close()
    assert [r["index"] for r in open_store(tmp_path).records()] == [2]


def test_damage_and_foreign_files(tmp_path):
    store = open_store(tmp_path)
    data = np.arange(8192, dtype=np.uint32).view(np.uint8)[:8192]
    for index in range(3):
        assert store.write(index, data, 1234 + index, bytes([index]) * 24)
    store.close()
    records = bytearray((tmp_path / "records").read_bytes())
    records[4096 + 64 + 20] ^= 1  # one bit of record 1's label
    (tmp_path / "records").write_bytes(bytes(records))
    with open(tmp_path / "slots", "r+b") as f:
        f.truncate(2 * 8192 + 100)  # slot 2 no longer lies wholly inside the slot file
    assert [r["index"] for r in open_store(tmp_path).records()] == [0]
    # a file written for another tag, slot size or label size is emptied when it opens
    for kwargs in ({"tag": b"tag-b"}, {"slot_bytes": 4096}, {"label_bytes": 28}):
        fresh = open_store(tmp_path, **kwargs)
        assert fresh.records() == []
        fresh.close()
        assert (tmp_path / "slots").stat().st_size == 0 and (tmp_path / "records").stat().st_size == 4096
    with pytest.raises(ValueError):
        open_store(tmp_path, slot_bytes=1000)  # not whole host pages
    with pytest.raises(ValueError):
        open_store(tmp_path, label_bytes=0)


def make(tier=Cache.MANUAL_TIER):
    pool = KvPool(pages=24, bytes_per_page=100, extent_pages=8, runway_pages=0, budget_pages=24)
    return pool, Cache(pool, tier, 16, 8)


def tokens(n, seed):
    return np.random.default_rng(seed).integers(0, 50000, size=n, dtype=np.uint32)


def fill_and_evict(pool, cache, prompts):
    """Publishes each prompt's full pages, then evicts every block to the tier (leaves first)."""
    for request, prompt in enumerate(prompts, start=1):
        cache.begin_request(request)
        full = len(prompt) // 32 * 32
        assert cache.ensure_tokens(request, full) == GRANTED
        for i, page in enumerate(cache.page_table(request)[0]):
            pool.set_page_content(page, request * 1000 + i)
        cache.publish(request, prompt, full)
        cache.end_request(request)
    while cache.reclaim_one():
        assert cache.complete_transfer(True)
        cache.poll_transfers()
    assert cache.snapshot()["resident_blocks"] == 0


def test_cache_persists_and_adopts_its_tier_copies(tmp_path):
    a, b = tokens(97, 1), tokens(65, 2)
    shared = np.concatenate([a[:64], tokens(33, 3)])  # shares a's first two pages
    pool, cache = make()
    fill_and_evict(pool, cache, [a, b, shared])
    blocks = cache.snapshot()["tier_blocks"]
    assert blocks == 3 + 2 + 1
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert cache.persist(store) == blocks
    store.close(); cache.close(); pool.close()

    # "the next process": new pool, cache and tier; the files are all that is left
    pool, cache = make()
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    records = store.records()
    assert len(records) == blocks and all(r["payload_bytes"] == 100 for r in records)
    label = np.frombuffer(records[0]["label"], dtype="<u8", count=5)
    assert label[0] == 1 and label[1] == 0 and (np.frombuffer(records[0]["label"], dtype="<u4", offset=40) == a[:32]).all()
    adopted = cache.adopt(store)
    assert adopted == {"blocks": blocks, "dropped": 0, "bytes": blocks * 100}
    with pytest.raises(RuntimeError):
        cache.adopt(store)  # only before anything else is in the cache
    for request, (prompt, pages) in enumerate([(a, 3), (b, 2), (shared, 3)], start=1):
        chain = cache.lookup(np.concatenate([prompt, [1]]))
        assert len(chain) == pages
        cache.begin_request(request)
        status, resume = cache.attach_prefix(request, chain)
        assert status == GRANTED and resume == pages * 32
        while cache.complete_transfer(True):
            cache.poll_transfers()
        assert not cache.restores_pending(request)
        table = cache.page_table(request)[0]
        want = [request * 1000 + i for i in range(pages)] if request < 3 else [1000, 1001, 3002]
        assert [pool.page_content(p) for p in table] == want
    # a block published now gets an id after every id a record named
    cache.begin_request(9)
    assert cache.ensure_tokens(9, 32) == GRANTED
    cache.publish(9, tokens(33, 9), 32)
    assert cache.lookup(tokens(33, 9)) == [blocks + 1]
    store.close(); cache.close(); pool.close()


def test_a_broken_chain_and_a_changed_payload_stay_behind(tmp_path):
    a = tokens(129, 5)
    pool, cache = make()
    fill_and_evict(pool, cache, [a])
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert cache.persist(store) == 4
    store.close(); cache.close(); pool.close()
    # lose the third block's record: everything below it has no chain any more
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    by_id = {int(np.frombuffer(r["label"], dtype="<u8", count=1)[0]): r["index"] for r in store.records()}
    assert sorted(by_id) == [1, 2, 3, 4]
    store.free(by_id[3])
    store.close()
    with open(tmp_path / "slots", "r+b") as f:  # and change one byte of the second block's payload
        f.seek(by_id[2] * 4096 + 50)
        byte = f.read(1)
        f.seek(by_id[2] * 4096 + 50)
        f.write(bytes([byte[0] ^ 0x40]))
    pool, cache = make()
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert cache.adopt(store) == {"blocks": 2, "dropped": 1, "bytes": 200}
    chain = cache.lookup(a)
    assert chain == [1, 2]
    cache.begin_request(1)
    assert cache.attach_prefix(1, chain)[0] == GRANTED
    assert cache.complete_transfer(True)   # block 1 arrives and matches its record
    assert cache.complete_transfer(True)   # block 2 arrives, but not the bytes its record names
    cache.poll_transfers()
    assert cache.snapshot()["failed_transfers"] == 1
    assert cache.lookup(a) == [1]          # a cache miss and nothing worse
    cache.end_request(1)
    # the dropped record was freed in the file: the next process no longer sees block 4
    store.close(); cache.close(); pool.close()
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert sorted(int(np.frombuffer(r["label"], dtype="<u8", count=1)[0]) for r in store.records()) == [1, 2]
    store.close()


def test_a_second_seal_is_written_beside_the_first_and_frees_it_afterwards(tmp_path):
    """Cache::persist writes the new set at indices the previous seal does not use, flushes, and only then frees the
    previous records (the reference frees a slot's record before its blocks: runtime/model/SlotFile.cpp:398-438): at no
    point do the files hold less than one whole seal. The sets alternate between the bottom of the file and the
    space above the previous set."""
    a = tokens(129, 5)
    pool, cache = make()
    fill_and_evict(pool, cache, [a])
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert cache.persist(store) == 4
    store.close()
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert sorted(r["index"] for r in store.records()) == [0, 1, 2, 3]
    assert cache.persist(store) == 4          # the second seal cannot go below the first: it goes above
    store.close()
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert sorted(r["index"] for r in store.records()) == [4, 5, 6, 7]
    assert cache.persist(store) == 4          # the third fits below the second again
    store.close()
    store = SlotStore(tmp_path / "slots", tmp_path / "records", b"manual", KV_BLOCK_LABEL_BYTES, 4096)
    assert sorted(r["index"] for r in store.records()) == [0, 1, 2, 3]
    cache.close(); pool.close()
    pool, cache = make()
    assert cache.adopt(store) == {"blocks": 4, "dropped": 0, "bytes": 400}
    assert cache.lookup(a) == [1, 2, 3, 4]
    store.close(); cache.close(); pool.close()


# ---- against the reference's OWN slot file, compiled in place (runtime/model/SlotFile.cpp into oracle/_ref) --------
needs_slot_file = pytest.mark.skipif(om.reference() is None or not hasattr(om.reference(), "ref_slotfile_write"),
                                     reason="the reference's slot file was not compiled here")
SLOT_BYTES, LABEL_BYTES, TAG = 32768, KV_BLOCK_LABEL_BYTES, b"int4/16x4x256/v1"


def reference_write(tmp_path, payloads, labels, payload_bytes):
    r = om.reference()
    flat = np.ascontiguousarray(np.stack(payloads), dtype=np.uint8)
    flat_labels = np.frombuffer(b"".join(labels), dtype=np.uint8).copy()
    tag = np.frombuffer(TAG, dtype=np.uint8).copy()
    return r.ref_slotfile_write(str(tmp_path / "slots").encode(), str(tmp_path / "records").encode(), tag.ctypes.data, len(TAG),
                                LABEL_BYTES, SLOT_BYTES, len(payloads), flat.ctypes.data, payload_bytes, flat_labels.ctypes.data)


def reference_read(tmp_path, capacity=16):
    r = om.reference()
    tag = np.frombuffer(TAG, dtype=np.uint8).copy()
    indices, sizes, sums = np.zeros(capacity, np.uint32), np.zeros(capacity, np.uint64), np.zeros(capacity, np.uint32)
    labels, payloads, ok = np.zeros((capacity, LABEL_BYTES), np.uint8), np.zeros((capacity, SLOT_BYTES), np.uint8), np.zeros(capacity, np.uint8)
    found = r.ref_slotfile_read(str(tmp_path / "slots").encode(), str(tmp_path / "records").encode(), tag.ctypes.data, len(TAG),
                                LABEL_BYTES, SLOT_BYTES, capacity, indices.ctypes.data, sizes.ctypes.data, sums.ctypes.data,
                                labels.ctypes.data, payloads.ctypes.data, SLOT_BYTES, ok.ctypes.data)
    assert found >= 0
    return [{"index": int(indices[i]), "payload_bytes": int(sizes[i]), "checksum": int(sums[i]), "label": labels[i].tobytes(),
             "payload": payloads[i, : int(sizes[i])].copy(), "ok": bool(ok[i])} for i in range(min(found, capacity))]


def some_slots(seed, count, payload_bytes):
    rng = np.random.default_rng(seed)
    payloads = [rng.integers(0, 256, payload_bytes, dtype=np.uint8) for _ in range(count)]
    labels = [kv_block_label(10 + i, 9 + i if i else 0, 100 + i, rng.integers(0, 50000, 32).tolist(), images=(i, 2 * i)) for i in range(count)]
    return payloads, labels


@needs_slot_file
def test_what_the_reference_writes_this_store_reads(tmp_path):
    payloads, labels = some_slots(3, 5, 30000)
    assert reference_write(tmp_path, payloads, labels, 30000) == 5
    store = SlotStore(tmp_path / "slots", tmp_path / "records", TAG, LABEL_BYTES, SLOT_BYTES)
    found = sorted(store.records(), key=lambda record: record["index"])
    assert [record["index"] for record in found] == list(range(5))
    for record, payload, label in zip(found, payloads, labels):
        assert record["payload_bytes"] == 30000 and record["label"] == label
        assert record["checksum"] == crc(payload.tobytes())     # the reference's worker took it while writing
        assert np.array_equal(store.read(record["index"], 30000), payload)
    store.close()


@needs_slot_file
def test_what_this_store_writes_the_reference_reads_and_verifies(tmp_path):
    payloads, labels = some_slots(4, 6, 20000)
    store = SlotStore(tmp_path / "slots", tmp_path / "records", TAG, LABEL_BYTES, SLOT_BYTES)
    for index, (payload, label) in enumerate(zip(payloads, labels)):
        assert store.write(index, payload, crc(payload.tobytes()), label)
    assert store.free(2)                                         # a freed slot has no record for the next process
    assert store.synchronize()
    store.close()
    found = sorted(reference_read(tmp_path), key=lambda record: record["index"])
    assert [record["index"] for record in found] == [0, 1, 3, 4, 5]
    for record in found:
        assert record["ok"], "the reference's first read of an adopted slot checks the payload against its record"
        assert record["payload_bytes"] == 20000 and record["label"] == labels[record["index"]]
        assert record["checksum"] == crc(payloads[record["index"]].tobytes())
        assert np.array_equal(record["payload"], payloads[record["index"]])
    # a payload that changed after its record was written fails the reference's check: a cache miss, nothing worse
    with open(tmp_path / "slots", "r+b") as slots:
        slots.seek(3 * SLOT_BYTES + 100)
        slots.write(b"\xff\xfe\xfd")
    damaged = {record["index"]: record["ok"] for record in reference_read(tmp_path)}
    assert damaged == {0: True, 1: True, 3: False, 4: True, 5: True}


@needs_slot_file
def test_both_write_the_same_bytes(tmp_path):
    payloads, labels = some_slots(5, 4, 32768)                   # whole slots: no tail for either side to zero differently
    (tmp_path / "theirs").mkdir(); (tmp_path / "mine").mkdir()
    assert reference_write(tmp_path / "theirs", payloads, labels, 32768) == 4
    store = SlotStore(tmp_path / "mine" / "slots", tmp_path / "mine" / "records", TAG, LABEL_BYTES, SLOT_BYTES)
    for index, (payload, label) in enumerate(zip(payloads, labels)):
        assert store.write(index, payload, crc(payload.tobytes()), label)
    assert store.synchronize()
    store.close()
    assert (tmp_path / "mine" / "slots").read_bytes() == (tmp_path / "theirs" / "slots").read_bytes()
    mine, theirs = (tmp_path / "mine" / "records").read_bytes(), (tmp_path / "theirs" / "records").read_bytes()
    used = 4096 + 4 * 192                                        # header area and four records
    assert mine[:used] == theirs[:used] and not any(mine[used:]) and not any(theirs[used:])
