"""Python handles over the host control plane (include/richkv_host.h): the page allocator
(engine::KvPool), the request / prefix cache with its eviction tier (engine::Cache subset) and the
operator plans (ops::PagedAttention). The objects live in C++ (richengine_b200/csrc/host)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib

GRANTED, DENIED, PENDING = 0, 1, 2
NO_PAGE = 0xFFFFFFFF
IMAGE_SPAN = np.dtype([("offset", "<u4"), ("tokens", "<u4"), ("grid_height", "<u4"), ("grid_width", "<u4"), ("digest_lo", "<u8"), ("digest_hi", "<u8")])


def image_spans(images):
    """rk_image_span records from (offset, tokens, grid_height, grid_width, digest_lo, digest_hi) tuples; (None, 0) for text."""
    if not images:
        return None, 0
    array = np.array([tuple(image) for image in images], dtype=IMAGE_SPAN)
    return array, len(array)


class KvPool:
    def __init__(self, *, pages=None, bytes_per_page=None, extent_pages=None, runway_pages=0, budget_pages=2 ** 62,
                 storage=None, stream=None):
        self._lib = lib.load()
        if storage is not None:
            self._handle = self._lib.rk_pool_create_device(storage.handle, runway_pages, stream)
            self.extent_pages = storage.extent_pages
        else:
            self._handle = self._lib.rk_pool_create_budget(pages, bytes_per_page, extent_pages, runway_pages, budget_pages)
            self.extent_pages = extent_pages
        if not self._handle:
            raise ValueError(self._lib.rk_last_error().decode())

    @property
    def handle(self):
        return self._handle

    def close(self):
        if self._handle:
            self._lib.rk_pool_destroy(self._handle)
            self._handle = None

    def set_budget(self, pages: int):
        self._lib.rk_pool_set_budget(self._handle, pages)

    def acquire(self, count: int):
        """The acquired page ids, or None when the pool could not grow."""
        out = (C.c_uint32 * max(count, 1))()
        got = self._lib.rk_pool_acquire(self._handle, count, out)
        if got == lib.REFUSED:
            return None
        lib.check(got, "rk_pool_acquire")
        return list(out[:got])

    def retain(self, page: int, prefix_owner=False):
        status = self._lib.rk_pool_retain(self._handle, page, int(prefix_owner))
        if status:
            raise RuntimeError(self._lib.rk_last_error().decode())

    def release(self, page: int, prefix_owner=False):
        status = self._lib.rk_pool_release(self._handle, page, int(prefix_owner))
        if status:
            raise RuntimeError(self._lib.rk_last_error().decode())

    def reclaim_empty_extents(self, keep_runway: bool, limit: int) -> int:
        return self._lib.rk_pool_reclaim_empty_extents(self._handle, int(keep_runway), limit)

    def compact_extent(self, fixed=()):
        fixed = np.ascontiguousarray(fixed, dtype=np.uint32)
        out = (C.c_uint32 * self.extent_pages)()
        first = self._lib.rk_pool_compact_extent(self._handle, fixed.ctypes.data, len(fixed), out)
        return None if first < 0 else (first, list(out))

    def snapshot(self) -> dict:
        out = (C.c_uint64 * 10)()
        self._lib.rk_pool_snapshot(self._handle, out)
        names = ["pages_allocated", "pages_free", "pages_active", "pages_prefix", "allocated_bytes", "reclaimable_bytes",
                 "extent_allocations", "extent_releases", "extent_compactions", "pages_moved"]
        return dict(zip(names, out))

    def page_content(self, page): return self._lib.rk_pool_page_content(self._handle, page)
    def set_page_content(self, page, tag): self._lib.rk_pool_set_page_content(self._handle, page, tag)


class Cache:
    NO_TIER, HOST_TIER, MANUAL_TIER = 0, 1, 2

    def __init__(self, pool: KvPool, tier_mode=0, slots=0, transfers=0):
        self._lib = lib.load()
        self.pool = pool
        self._handle = self._lib.rk_cache_create(pool.handle, tier_mode, slots, transfers)
        if not self._handle:
            raise ValueError(self._lib.rk_last_error().decode())

    def close(self):
        if self._handle:
            self._lib.rk_cache_destroy(self._handle)
            self._handle = None

    def _check(self, status, where):
        if status < 0:
            raise RuntimeError(f"{where}: {self._lib.rk_last_error().decode()}")
        return status

    def begin_request(self, request): self._check(self._lib.rk_cache_begin_request(self._handle, request), "begin_request")
    def end_request(self, request): self._check(self._lib.rk_cache_end_request(self._handle, request), "end_request")
    def ensure_tokens(self, request, tokens) -> int: return self._check(self._lib.rk_cache_ensure_tokens(self._handle, request, tokens), "ensure_tokens")

    def page_table(self, request):
        revision, first = C.c_uint64(), C.c_uint32()
        count = self._check(self._lib.rk_cache_page_table(self._handle, request, None, 0, C.byref(revision), C.byref(first)), "page_table")
        out = (C.c_uint32 * max(count, 1))()
        self._lib.rk_cache_page_table(self._handle, request, out, count, None, None)
        return list(out[:count]), revision.value, first.value

    def publish(self, request, tokens, committed, images=None):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        spans, count = image_spans(images)
        self._check(self._lib.rk_cache_publish(self._handle, request, t.ctypes.data, len(t), committed,
                                               spans.ctypes.data if count else None, count), "publish")

    def lookup(self, prompt, images=None):
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = (C.c_uint64 * (len(t) // 32 + 1))()
        spans, n = image_spans(images)
        count = self._check(self._lib.rk_cache_lookup(self._handle, t.ctypes.data, len(t), out, len(out), spans.ctypes.data if n else None, n), "lookup")
        return list(out[:count])

    def attach_prefix(self, request, blocks):
        b = (C.c_uint64 * max(len(blocks), 1))(*blocks)
        resume = C.c_uint32()
        status = self._check(self._lib.rk_cache_attach_prefix(self._handle, request, b, len(blocks), C.byref(resume)), "attach_prefix")
        return status, resume.value

    def restores_pending(self, request) -> bool: return bool(self._check(self._lib.rk_cache_restores_pending(self._handle, request), "restores_pending"))
    def restore_status(self, request) -> int:
        """0 = nothing to wait for, 1 = pending, 2 = a read failed (Cache::kvRestoreStatus)."""
        return self._check(self._lib.rk_cache_restore_status(self._handle, request), "restore_status")

    def set_state_coupled(self, coupled=True): self._lib.rk_cache_set_state_coupled(self._handle, int(coupled))
    def manual_tier_plain_limits(self, plain=True): self._lib.rk_cache_manual_tier_plain_limits(self._handle, int(plain))
    def manual_tier_set(self, transfer_limit, writable=True): self._lib.rk_cache_manual_tier_set(self._handle, transfer_limit, int(writable))

    def tier_counters(self) -> dict:
        out = (C.c_uint64 * 6)()
        self._lib.rk_cache_tier_counters(self._handle, out)
        return dict(zip(["demotions_refused", "replaced_copies", "cancelled_restores", "pending_pages", "demotions_landed", "restores_landed"],
                        [int(x) for x in out]))

    def fork(self, parent, child, committed) -> int: return self._check(self._lib.rk_cache_fork(self._handle, parent, child, committed), "fork")
    def truncate(self, request, committed, scratch) -> int: return self._check(self._lib.rk_cache_truncate(self._handle, request, committed, scratch), "truncate")
    def reclaim_one(self) -> bool: return bool(self._check(self._lib.rk_cache_reclaim_one(self._handle), "reclaim_one"))
    def reclaim_for_pages(self, pages) -> int: return self._lib.rk_cache_reclaim_for_pages(self._handle, pages)
    def poll_transfers(self): self._lib.rk_cache_poll_transfers(self._handle)
    def compact_extent(self) -> bool: return bool(self._check(self._lib.rk_cache_compact_extent(self._handle), "compact_extent"))
    def complete_transfer(self, success=True) -> bool: return bool(self._lib.rk_cache_complete_transfer(self._handle, int(success)))
    def fail_next_transfers(self, count): self._lib.rk_cache_fail_next_transfers(self._handle, count)

    # ---- composite states and the reclaim order they impose (engine::StateCache subset, Cache::evictOne) ----
    def block_at(self, request, tokens) -> int: return self._check(self._lib.rk_cache_block_at(self._handle, request, tokens), "block_at")
    def publish_state(self, block, size, checkpoint=False): self._check(self._lib.rk_cache_state_publish(self._handle, block, size, int(checkpoint)), "publish_state")
    def publish_stored_state(self, block, size, checkpoint=False): self._check(self._lib.rk_cache_state_publish_stored(self._handle, block, size, int(checkpoint)), "publish_stored_state")
    def use_state(self, block): self._check(self._lib.rk_cache_state_use(self._handle, block, 1), "use_state")
    def unuse_state(self, block): self._check(self._lib.rk_cache_state_use(self._handle, block, 0), "unuse_state")
    def pin_state(self, block): self._check(self._lib.rk_cache_state_pin(self._handle, block, 1), "pin_state")
    def unpin_state(self, block): self._check(self._lib.rk_cache_state_pin(self._handle, block, 0), "unpin_state")

    def state_info(self, block) -> dict:
        out = (C.c_uint64 * 7)()
        self._check(self._lib.rk_cache_state_info(self._handle, block, out), "state_info")
        return dict(zip(["contains", "ordinary", "in_use", "bytes", "kv_needed", "kv_needed_in_use", "resident"], [int(x) for x in out]))

    def state_summary(self) -> dict:
        out = (C.c_uint64 * 4)()
        self._check(self._lib.rk_cache_state_summary(self._handle, out), "state_summary")
        return dict(zip(["states", "bytes", "evictable", "resume_point"], [int(x) for x in out]))

    def evict_one(self, up_to_in_use=True, keep_resume_point=False, pages_only=False) -> dict:
        out = (C.c_uint64 * 4)()
        self._check(self._lib.rk_cache_evict_one(self._handle, int(up_to_in_use), int(keep_resume_point), int(pages_only), out), "evict_one")
        return dict(zip(["progress", "pending", "evicted_state", "state_bytes"], [int(x) for x in out]))

    RELEASE_EXTENTS, KEEP_EXTENTS, REUSE_PAGES = 0, 1, 2

    def reclaim_step(self, mode=0, up_to_in_use=True, keep_resume_point=False, keep_runway=False) -> dict:
        """Cache::reclaimOne(mode, ...): an empty extent, else a gathered one, else one victim."""
        out = (C.c_uint64 * 4)()
        self._check(self._lib.rk_cache_reclaim_step(self._handle, mode, int(up_to_in_use), int(keep_resume_point), int(keep_runway), out), "reclaim_step")
        return dict(zip(["progress", "pending", "evicted_state", "bytes"], [int(x) for x in out]))

    def evict_all(self) -> dict:
        out = (C.c_uint64 * 2)()
        self._check(self._lib.rk_cache_evict_all(self._handle, out), "evict_all")
        return {"progress": bool(out[0]), "bytes": int(out[1])}

    def lookup_state(self, prompt, record=False, probe=None, images=None) -> dict:
        """Cache::lookup with states: the chain, the deepest state on it (pinned: unpin_state when done), where the
        request resumes, a junction worth a state, a state that was lost. A current Probe's chain is reused."""
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        blocks = (C.c_uint64 * (len(t) // 32 + 1))()
        out = (C.c_uint64 * 5)()
        spans, n = image_spans(images)
        count = self._check(self._lib.rk_cache_lookup_state(self._handle, t.ctypes.data, len(t), blocks, len(blocks), out, int(record),
                                                            probe._handle if probe is not None else None,
                                                            spans.ctypes.data if n else None, n), "lookup_state")
        return {"blocks": list(blocks[:count]), "kv_boundary": int(out[0]), "state_block": int(out[1]), "resume_boundary": int(out[2]),
                "junction_boundary": int(out[3]), "lost_state": bool(out[4])}

    def lookup_counters(self) -> dict:
        out = (C.c_uint64 * 4)()
        self._check(self._lib.rk_cache_lookup_counters(self._handle, out), "lookup_counters")
        return dict(zip(["kv_hit_tokens", "lazy_junctions", "lost_state_misses", "probe_hashed_blocks"], [int(x) for x in out]))

    def probe(self, prompt, images=None) -> "Probe":
        """Cache::probe: what a scheduler keeps per waiting request between admission passes."""
        return Probe(self, prompt, images)

    def reclaim_one_state(self, checkpoints_only=False, for_block=0) -> bool:
        return bool(self._check(self._lib.rk_cache_reclaim_one_state(self._handle, int(checkpoints_only), for_block), "reclaim_one_state"))

    def snapshot(self) -> dict:
        out = (C.c_uint64 * 10)()
        self._lib.rk_cache_snapshot(self._handle, out)
        names = ["requests", "resident_blocks", "tier_blocks", "transfers", "demotions", "restores", "failed_transfers",
                 "evicted_blocks", "fork_copies", "truncated_pages"]
        return dict(zip(names, out))

    def persist(self, store: "SlotStore") -> int:
        """Seals every landed tier copy into the store (payload, its device-computed CRC-32C, its KvBlockLabel)."""
        return self._check(self._lib.rk_cache_persist(self._handle, store.handle), "persist")

    def adopt(self, store: "SlotStore") -> dict:
        """On an empty cache: takes back what an earlier process sealed. {blocks, dropped, bytes}."""
        out = (C.c_uint64 * 3)()
        self._check(self._lib.rk_cache_adopt(self._handle, store.handle, out), "adopt")
        return {"blocks": out[0], "dropped": out[1], "bytes": out[2]}

    def adopt_restore_points(self, store: "SlotStore", states) -> dict:
        """On an empty cache, the reference's rule: each stored state comes back with its whole chain, a block only for
        a state. states = [(label bytes of a StateLabel, size in bytes)]. {blocks, dropped, bytes, states}."""
        labels = C.create_string_buffer(b"".join(label for label, _ in states), max(1, STATE_LABEL_BYTES * len(states)))
        sizes = (C.c_uint64 * max(1, len(states)))(*[size for _, size in states])
        out = (C.c_uint64 * 4)()
        self._check(self._lib.rk_cache_adopt_restore_points(self._handle, store.handle, labels, sizes, len(states), out), "adopt_restore_points")
        return {"blocks": out[0], "dropped": out[1], "bytes": out[2], "states": out[3]}

    def state_labels(self):
        """[(StateLabel bytes, size)] of every stored state, as a clean stop records them."""
        count = self._check(self._lib.rk_cache_state_labels(self._handle, None, None, 0), "state_labels")
        labels = C.create_string_buffer(max(1, STATE_LABEL_BYTES * count))
        sizes = (C.c_uint64 * max(1, count))()
        self._check(self._lib.rk_cache_state_labels(self._handle, labels, sizes, count), "state_labels")
        return [(labels.raw[i * STATE_LABEL_BYTES:(i + 1) * STATE_LABEL_BYTES], int(sizes[i])) for i in range(count)]

    def block_state(self, block):
        out = (C.c_uint64 * 5)()
        if self._lib.rk_cache_block_state(self._handle, block, out) < 0:
            return None
        return {"page": out[0], "tier_copy": bool(out[1]), "transferring": bool(out[2]), "last_used": out[3], "poisoned": bool(out[4])}


STATE_LABEL_BYTES = 24  # engine::StateLabel: block, lastUsed (u64 each), tokens, checkpoint (u32 each)
KV_BLOCK_LABEL_BYTES = 168  # engine::KvBlockLabel: id, parent, lastUsed, images lo/hi (u64 each), 32 token ids (u32)


class Probe:
    """The scheduling probe of a waiting request (CacheProbe, runtime/engine/cache/Cache.hpp:38-52): pins nothing,
    touches no recency, counts no hit; refresh() hashes only what a change of the block graph made necessary."""

    def __init__(self, cache: Cache, prompt, images=None):
        self._cache, self._lib = cache, cache._lib
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        spans, n = image_spans(images)
        self._handle = self._lib.rk_cache_probe_create(cache._handle, t.ctypes.data, len(t), spans.ctypes.data if n else None, n)
        if not self._handle:
            raise RuntimeError(f"probe: {self._lib.rk_last_error().decode()}")

    def refresh(self, prompt, cache: Cache = None, images=None):
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        owner = cache if cache is not None else self._cache
        spans, n = image_spans(images)
        owner._check(self._lib.rk_cache_probe_refresh(owner._handle, self._handle, t.ctypes.data, len(t), spans.ctypes.data if n else None, n), "probe_refresh")

    def _info(self):
        out = (C.c_uint64 * 2)()
        self._cache._check(self._lib.rk_cache_probe_info(self._handle, out), "probe_info")
        return int(out[0]), int(out[1])

    @property
    def cached_tokens(self) -> int: return self._info()[0]

    @property
    def matched_blocks(self) -> int: return self._info()[1]

    def close(self):
        if self._handle:
            self._lib.rk_cache_probe_destroy(self._handle)
            self._handle = None

    def __del__(self):
        self.close()


def state_label(block, last_used, tokens, checkpoint=False) -> bytes:
    return np.array([block, last_used], dtype="<u8").tobytes() + np.array([tokens, int(checkpoint)], dtype="<u4").tobytes()


def kv_block_label(block_id, parent, last_used, tokens, images=(0, 0)) -> bytes:
    assert len(tokens) == 32
    return np.array([block_id, parent, last_used, images[0], images[1]], dtype="<u8").tobytes() + np.asarray(tokens, dtype="<u4").tobytes()


class SlotStore:
    """Slots in one file and their records beside it, in the reference's byte format (model::SlotFile, persistent)."""

    def __init__(self, slots_path, records_path, tag: bytes, label_bytes: int, slot_bytes: int):
        self._lib = lib.load()
        self.label_bytes, self.slot_bytes = label_bytes, slot_bytes
        tag_buffer = C.create_string_buffer(tag, max(len(tag), 1))
        self.handle = self._lib.rk_slot_store_open(str(slots_path).encode(), str(records_path).encode(), tag_buffer, len(tag),
                                                   label_bytes, slot_bytes)
        if not self.handle:
            raise ValueError(self._lib.rk_last_error().decode())

    def close(self):
        if self.handle:
            self._lib.rk_slot_store_close(self.handle)
            self.handle = None

    def records(self):
        found = []
        for at in range(self._lib.rk_slot_store_record_count(self.handle)):
            index, size, checksum = C.c_uint32(), C.c_uint64(), C.c_uint32()
            label = C.create_string_buffer(self.label_bytes)
            self._lib.rk_slot_store_record(self.handle, at, C.byref(index), C.byref(size), C.byref(checksum), label)
            found.append({"index": index.value, "payload_bytes": size.value, "checksum": checksum.value, "label": label.raw})
        return found

    def write(self, index, payload: np.ndarray, checksum: int, label: bytes) -> bool:
        payload = np.ascontiguousarray(payload, dtype=np.uint8)
        status = self._lib.rk_slot_store_write(self.handle, index, payload.ctypes.data, payload.size, checksum,
                                               C.create_string_buffer(label, len(label)))
        if status == lib.INVALID:
            raise ValueError(self._lib.rk_last_error().decode())
        return status == lib.OK

    def read(self, index, size) -> np.ndarray | None:
        out = np.empty(size, np.uint8)
        return out if self._lib.rk_slot_store_read(self.handle, index, out.ctypes.data, size) == lib.OK else None

    def free(self, index) -> bool: return self._lib.rk_slot_store_free(self.handle, index) == lib.OK
    def synchronize(self) -> bool: return self._lib.rk_slot_store_synchronize(self.handle) == lib.OK


def verify_plan(lanes, query_heads, layout, history, tree=False, row_capacity=0, ctas=0):
    """(pipeline names, numbers): out[0] splits, [1:5] lane splits, ..., [13] row capacity, [14] streaming
    decode, [15] tcgen05 window kernel. `ctas` 0 = the device's SM count (no device: the reference plan)."""
    library = lib.load()
    names = C.create_string_buffer(512)
    out = (C.c_uint64 * 16)()
    h = (C.c_uint32 * lanes)(*history)
    status = library.rk_plan_verify(lanes, query_heads, layout.attention_layers, layout.kv_heads, layout.head_dimension,
                                    layout.format, h, int(tree), row_capacity, ctas, names, 512, out)
    if status:
        raise ValueError(library.rk_last_error().decode())
    return names.value.decode().split("\n"), list(out[:16])


def window_splits(lanes, kv_heads, visible_tokens, ctas=0):
    """Split count of one lane for the tcgen05 window kernel (PagedAttention::windowSplits); ctas 0 = this device."""
    value = lib.load().rk_plan_window_splits(lanes, kv_heads, visible_tokens, ctas)
    if value <= 0:
        raise ValueError(lib.load().rk_last_error().decode())
    return int(value)


def prefill_plan(rows, query_heads, layout):
    library = lib.load()
    names = C.create_string_buffer(512)
    out = (C.c_uint64 * 16)()
    status = library.rk_plan_prefill(rows, query_heads, layout.attention_layers, layout.kv_heads, layout.head_dimension,
                                     layout.format, names, 512, out)
    if status:
        raise ValueError(library.rk_last_error().decode())
    return names.value.decode().split("\n"), list(out[:10])
