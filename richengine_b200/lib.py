"""ctypes binding of librichkv.so — the C ABI declared in include/richkv.h.

Loading never falls back to anything: a missing library raises, so a caller can
not run on a silent CPU path. Build it with `python -m richengine_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# RICHKV_LIBRARY names another build of the same library (e.g. a profiling build).
LIBRARY_PATH = Path(os.environ.get("RICHKV_LIBRARY") or Path(__file__).resolve().parent / "librichkv.so")

OK, INVALID, CUDA_ERROR, UNSUPPORTED, REFUSED, TIMEOUT = 0, -1, -2, -3, -4, -5


class KvLayer(C.Structure):
    _fields_ = [("extent_pages", C.c_uint32), ("offset", C.c_uint32)]


class ChunkParams(C.Structure):
    _fields_ = [("committed_tokens", C.c_uint32), ("chunk_tokens", C.c_uint32), ("chunk_stride", C.c_uint32),
                ("page_table_entries", C.c_uint32), ("kv", KvLayer)]


class PrefillParams(C.Structure):
    _fields_ = [("committed_tokens", C.c_uint32), ("rows", C.c_uint32), ("chunk_stride", C.c_uint32),
                ("page_table_entries", C.c_uint32), ("kv", KvLayer), ("split_count", C.c_uint32),
                ("score_scale", C.c_float)]


class VerifyParams(C.Structure):
    _fields_ = [("committed_tokens", C.c_uint32), ("page_table_entries", C.c_uint32), ("kv", KvLayer),
                ("split_count", C.c_uint32), ("slot_splits", C.c_uint32), ("active_rows", C.c_uint32),
                ("row_capacity", C.c_uint32), ("score_scale", C.c_float)]


class PageCopy(C.Structure):
    _fields_ = [("from_page", C.c_uint32), ("to_page", C.c_uint32)]


class DecodePlan(C.Structure):
    """rk_decode_plan (include/richkv.h)."""
    _fields_ = [("lanes", C.c_uint32), ("ctas", C.c_uint32), ("max_segments", C.c_uint32), ("reserved", C.c_uint32),
                ("partials_bytes", C.c_uint64), ("statistics_bytes", C.c_uint64), ("descriptor_bytes", C.c_uint64)]


class VerifyBuffers(C.Structure):
    """rk_verify_buffers (include/richkv_host.h)."""
    _fields_ = [("chunk_keys", C.c_void_p), ("chunk_values", C.c_void_p), ("queries", C.c_void_p), ("output", C.c_void_p),
                ("partials", C.c_void_p), ("statistics", C.c_void_p), ("descriptors", C.c_void_p), ("status", C.c_void_p),
                ("page_tables", C.c_void_p), ("tree_masks", C.c_void_p), ("partials_bytes", C.c_uint64),
                ("statistics_bytes", C.c_uint64)]


assert C.sizeof(ChunkParams) == 24 and C.sizeof(PrefillParams) == 32 and C.sizeof(VerifyParams) == 36

u32, u64, i32, i64, vp, f32p = C.c_uint32, C.c_uint64, C.c_int, C.c_int64, C.c_void_p, C.c_void_p

# name -> (restype, argtypes). Every symbol include/richkv.h declares is listed
# here; tests check the library exports each of them.
SIGNATURES = {
    "rk_last_error": (C.c_char_p, []),
    "rk_extent_alignment_pages": (u32, [u32, u32, u32]),
    # kernels
    "rk_store_verify": (i32, [u32, u32, u32, u32, u32, vp, vp, vp, vp, KvLayer, vp]),
    "rk_store_chunk": (i32, [u32, u32, u32, vp, vp, vp, C.POINTER(ChunkParams), vp]),
    "rk_attention_verify_split": (i32, [u32, u32, u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, KvLayer, vp]),
    "rk_attention_verify_split_tc": (i32, [vp, u32, u32, u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, KvLayer, vp, vp]),
    "rk_attention_verify_probe_timeout": (i32, [vp, u32, u32, u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, KvLayer, vp, u32, u32, vp]),
    "rk_attention_verify_reduce": (i32, [u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp]),
    "rk_qkv_prepare": (i32, [u32, u32, u32, u32, u32, vp, vp, vp, i32, vp, vp, C.c_float, vp, vp, vp, vp]),
    "rk_qkv_prepare_store": (i32, [u32, u32, u32, u32, u32, u32, vp, vp, vp, i32, vp, vp, C.c_float, vp, vp, vp, KvLayer, vp]),
    "rk_crc32c_pages": (i32, [vp, u64, u64, u32, vp, u32, vp]),
    "rk_crc32c_host": (u32, [vp, u64, u32]),
    "rk_attention_verify_reduce_gate": (i32, [u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, vp]),
    "rk_attention_prefill_split": (i32, [u32, u32, u32, u32, vp, vp, vp, vp, C.POINTER(PrefillParams), vp]),
    "rk_attention_prefill_split_tc": (i32, [vp, u32, u32, u32, u32, vp, vp, vp, vp, C.POINTER(PrefillParams), vp, vp]),
    "rk_attention_prefill_reduce": (i32, [u32, u32, u32, vp, vp, vp, vp, C.POINTER(PrefillParams), vp]),
    "rk_copy_pages": (i32, [u32, u32, u32, u32, u32, vp, vp, u32, vp]),
    "rk_pack_pages": (i32, [u32, u32, u32, u32, u32, vp, vp, u32, vp]),
    "rk_unpack_pages": (i32, [u32, u32, u32, u32, u32, vp, vp, u32, vp]),
    "rk_tree_compact": (i32, [u32, u32, u32, u32, vp, vp, KvLayer, vp, vp, vp]),
    # streaming decode attention
    "rk_decode_plan_make": (i32, [u32, u32, u32, u32, u32, u32, C.POINTER(DecodePlan)]),
    "rk_window_create": (vp, [u64, u64]),
    "rk_window_destroy": (None, [vp]),
    "rk_attention_decode": (i32, [vp, C.POINTER(DecodePlan), u32, vp, vp, vp, vp, vp, vp, vp, vp, KvLayer, vp]),
    "rk_attention_decode_shard": (i32, [vp, C.POINTER(DecodePlan), u32, vp, vp, vp, vp, vp, vp, vp, KvLayer, vp]),
    "rk_attention_merge_shards": (i32, [u32, u32, u32, u32, u32, vp, vp, vp, vp]),
    "rk_exchange_create": (vp, [u32, u32, u32, vp]),
    "rk_exchange_connect": (i32, [vp, vp]),
    "rk_exchange_destroy": (None, [vp]),
    "rk_attention_decode_exchange": (i32, [vp, C.POINTER(DecodePlan), u32, vp, vp, vp, vp, vp, vp, vp, vp, KvLayer, vp, i32, vp]),
    "rk_attention_decode_static": (i32, [vp, u32, u32, vp, vp, vp, vp, vp, KvLayer, vp]),
    "rk_attention_decode_status": (i32, [C.POINTER(DecodePlan), vp, vp]),
    "rk_attention_decode_static_status": (i32, [vp]),
    "rk_attention_decode_probe_timeout": (i32, [vp, C.POINTER(DecodePlan), u32, vp, vp, vp, vp, vp, vp, vp, KvLayer, u32, u32, vp]),
    "rk_stage_decode_rows": (i32, [u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, vp]),
    "rk_gather_decode_rows": (i32, [u32, u32, u32, u32, vp, vp, vp]),
    "rk_session_create": (vp, [u32, u32, u32, u32, u32, vp, vp, u32, u32]),
    "rk_session_destroy": (None, [vp]),
    "rk_session_step_host": (i32, [vp, u32, vp, vp, vp, vp, vp, vp, vp, vp]),
    "rk_session_finish_host": (i32, [vp, vp]),
    "rk_session_status": (i32, [vp, vp]),
    # storage
    "rk_storage_create": (vp, [u32, u32, u32, u32, u32, u32]),
    "rk_storage_destroy": (None, [vp]),
    "rk_storage_allocate_extent": (i32, [vp, u32]),
    "rk_storage_release_extent": (i32, [vp, u32]),
    "rk_storage_set_budget": (None, [vp, u64]),
    "rk_storage_page_count": (u32, [vp]),
    "rk_storage_extent_pages": (u32, [vp]),
    "rk_storage_bytes_per_page": (u64, [vp]),
    "rk_storage_extent_bytes": (u64, [vp]),
    "rk_storage_allocated_bytes": (u64, [vp]),
    "rk_storage_is_allocated": (i32, [vp, u32]),
    "rk_storage_window": (None, [vp, C.POINTER(u64), C.POINTER(u64)]),
    "rk_storage_layers": (u32, [vp, C.POINTER(KvLayer), u32]),
    "rk_storage_entry": (u64, [vp, u32]),
    "rk_storage_read_extent": (i32, [vp, u32, u64, vp, u64]),
    "rk_storage_write_extent": (i32, [vp, u32, u64, vp, u64]),
    "rk_storage_write_entries": (i32, [vp, vp, u32, u32, vp, u32, vp]),
    "rk_storage_copy_pages": (i32, [vp, vp, u32, vp]),
    "rk_storage_pack_pages": (i32, [vp, vp, u32, vp, i32, vp]),
    "rk_storage_seal_pages": (i32, [vp, vp, u32, vp, vp, vp]),
    # pinned-host tier
    "rk_tier_create": (vp, [vp, u32, u32]),
    "rk_tier_destroy": (None, [vp]),
    "rk_tier_slot_bytes": (u64, [vp]),
    "rk_tier_writable": (i32, [vp]),
    "rk_tier_can_demote": (i32, [vp]),
    "rk_tier_can_restore": (i32, [vp]),
    "rk_tier_acquire_slot": (i64, [vp]),
    "rk_tier_release_slot": (None, [vp, u32]),
    "rk_tier_fail_next": (None, [vp, u32]),
    "rk_tier_slot_checksum": (u32, [vp, u32]),
    "rk_tier_adopt_slot": (i64, [vp, vp, u64, u32]),
    "rk_tier_slot_host_pointer": (vp, [vp, u32]),
    "rk_tier_demote": (i32, [vp, u32, u32, vp]),
    "rk_tier_restore": (i32, [vp, u32, u32, vp]),
    "rk_tier_poll": (i32, [vp]),
    "rk_tier_transfer_ready": (i32, [vp, u32]),
    "rk_tier_transfer_finish": (i32, [vp, u32]),
    "rk_tier_drain": (i32, [vp]),
    # host control plane (include/richkv_host.h)
    "rk_pool_create_budget": (vp, [u32, u64, u32, u32, u64]),
    "rk_pool_create_device": (vp, [vp, u32, vp]),
    "rk_pool_destroy": (None, [vp]),
    "rk_pool_set_budget": (None, [vp, u64]),
    "rk_pool_acquire": (i32, [vp, u32, vp]),
    "rk_pool_retain": (i32, [vp, u32, i32]),
    "rk_pool_release": (i32, [vp, u32, i32]),
    "rk_pool_reclaim_empty_extents": (u64, [vp, i32, u32]),
    "rk_pool_compact_extent": (i64, [vp, vp, u32, vp]),
    "rk_pool_snapshot": (None, [vp, vp]),
    "rk_pool_page_content": (u64, [vp, u32]),
    "rk_pool_set_page_content": (None, [vp, u32, u64]),
    "rk_cache_create": (vp, [vp, i32, u32, u32]),
    "rk_cache_destroy": (None, [vp]),
    "rk_cache_begin_request": (i32, [vp, u64]),
    "rk_cache_end_request": (i32, [vp, u64]),
    "rk_cache_ensure_tokens": (i32, [vp, u64, u64]),
    "rk_cache_page_table": (i64, [vp, u64, vp, u32, C.POINTER(u64), C.POINTER(u32)]),
    "rk_block_image_identity": (None, [u64, u32, vp, u32, vp]),
    "rk_cache_publish": (i32, [vp, u64, vp, u32, u32, vp, u32]),
    "rk_cache_lookup": (i64, [vp, vp, u32, vp, u32, vp, u32]),
    "rk_cache_attach_prefix": (i32, [vp, u64, vp, u32, C.POINTER(u32)]),
    "rk_cache_restores_pending": (i32, [vp, u64]),
    "rk_cache_restore_status": (i32, [vp, u64]),
    "rk_cache_reclaim_step": (i32, [vp, i32, i32, i32, i32, vp]),
    "rk_cache_evict_all": (i32, [vp, vp]),
    "rk_cache_set_state_coupled": (None, [vp, i32]),
    "rk_cache_manual_tier_set": (None, [vp, u32, i32]),
    "rk_cache_manual_tier_plain_limits": (None, [vp, i32]),
    "rk_cache_tier_counters": (None, [vp, vp]),
    "rk_cache_fork": (i32, [vp, u64, u64, u32]),
    "rk_cache_truncate": (i64, [vp, u64, u32, u32]),
    "rk_cache_reclaim_one": (i32, [vp]),
    "rk_cache_reclaim_for_pages": (u32, [vp, u32]),
    "rk_cache_poll_transfers": (None, [vp]),
    "rk_cache_compact_extent": (i32, [vp]),
    "rk_cache_complete_transfer": (i32, [vp, i32]),
    "rk_cache_fail_next_transfers": (None, [vp, u32]),
    "rk_cache_snapshot": (None, [vp, vp]),
    "rk_cache_block_state": (i32, [vp, u64, vp]),
    "rk_cache_block_at": (i64, [vp, u64, u32]),
    "rk_cache_state_publish": (i32, [vp, u64, u64, i32]),
    "rk_cache_state_publish_stored": (i32, [vp, u64, u64, i32]),
    "rk_cache_state_use": (i32, [vp, u64, i32]),
    "rk_cache_state_pin": (i32, [vp, u64, i32]),
    "rk_cache_state_info": (i32, [vp, u64, vp]),
    "rk_cache_state_summary": (i32, [vp, vp]),
    "rk_cache_evict_one": (i32, [vp, i32, i32, i32, vp]),
    "rk_cache_reclaim_one_state": (i32, [vp, i32, u64]),
    "rk_cache_lookup_state": (i64, [vp, vp, u32, vp, u32, vp, i32, vp, vp, u32]),
    "rk_cache_probe_create": (vp, [vp, vp, u32, vp, u32]),
    "rk_cache_probe_refresh": (i32, [vp, vp, vp, u32, vp, u32]),
    "rk_cache_probe_info": (i32, [vp, vp]),
    "rk_cache_probe_destroy": (None, [vp]),
    "rk_cache_lookup_counters": (i32, [vp, vp]),
    "rk_slot_store_open": (vp, [C.c_char_p, C.c_char_p, vp, u32, u32, u64]),
    "rk_slot_store_close": (None, [vp]),
    "rk_slot_store_record_count": (u32, [vp]),
    "rk_slot_store_record": (i32, [vp, u32, vp, vp, vp, vp]),
    "rk_slot_store_write": (i32, [vp, u32, vp, u64, u32, vp]),
    "rk_slot_store_read": (i32, [vp, u32, vp, u64]),
    "rk_slot_store_free": (i32, [vp, u32]),
    "rk_slot_store_synchronize": (i32, [vp]),
    "rk_slot_record_bytes": (u64, [u32]),
    "rk_slot_record_encode": (i32, [u32, u64, u32, vp, vp]),
    "rk_slot_records_header": (i64, [u64, u32, vp, u32, vp, u32]),
    "rk_cache_persist": (i64, [vp, vp]),
    "rk_cache_adopt": (i32, [vp, vp, vp]),
    "rk_cache_adopt_restore_points": (i32, [vp, vp, vp, vp, u32, vp]),
    "rk_cache_state_labels": (i64, [vp, vp, vp, u32]),
    "rk_plan_window_splits": (i32, [u32, u32, u32, u32]),
    "rk_plan_verify": (i32, [u32, u32, u32, u32, u32, u32, vp, i32, u32, u32, C.c_char_p, C.c_size_t, vp]),
    "rk_plan_prefill": (i32, [u32, u32, u32, u32, u32, u32, C.c_char_p, C.c_size_t, vp]),
    "rk_plan_workspaces": (i32, [u32, u32, u32, u32, u32, u32, u32, vp]),
    "rk_op_verify_plan": (vp, [u32, u32, u32, u32, u32, u32, vp, i32, u32, u32]),
    "rk_op_prefill_plan": (vp, [u32, u32, u32, u32, u32, u32]),
    "rk_op_plan_destroy": (None, [vp]),
    "rk_op_plan_workspace": (i32, [vp, vp]),
    "rk_op_plan_lane_splits": (u32, [vp, u32]),
    "rk_op_add_prefill_store": (i32, [vp, KvLayer, vp, vp, vp, C.POINTER(ChunkParams), u32, u32, u32, u32]),
    "rk_op_add_prefill": (i32, [vp, KvLayer, vp, vp, vp, vp, u64, u64, vp, C.POINTER(ChunkParams), vp, vp, vp]),
    "rk_op_add_verify": (i32, [vp, KvLayer, C.POINTER(VerifyBuffers), vp, vp, vp, vp]),
    "rk_op_add_verify_tree_compact": (i32, [vp, KvLayer, vp, vp, vp, vp, u32, u32, u32, u32, u32]),
    "rk_chunk_validation_error": (C.c_char_p, [u32, u32, u32, u32]),
}

_library = None


def load() -> C.CDLL:
    """Loads librichkv.so and types its entry points. Raises if it is missing."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build the CUDA library with `python -m richengine_b200.build`; "
            "there is no CPU fallback")
    library = C.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(library, name)  # AttributeError names the missing symbol
        function.restype = restype
        function.argtypes = argtypes
    _library = library
    return library


class RichKvError(RuntimeError):
    def __init__(self, status: int, where: str):
        text = load().rk_last_error().decode(errors="replace")
        super().__init__(f"{where}: status {status}: {text}")
        self.status = status


def check(status: int, where: str) -> int:
    if status < 0:
        raise RichKvError(status, where)
    return status
