"""ctypes access to the CPU checker (oracle/). Test infrastructure only."""
import ctypes as C
from pathlib import Path

import numpy as np

from richengine_b200.lib import ChunkParams, KvLayer, VerifyParams

ROOT = Path(__file__).resolve().parent.parent
ORACLE_PATH = ROOT / "oracle" / "_build" / "librk_oracle.so"
REFERENCE_PATH = ROOT / "oracle" / "_ref" / "librk_ref.so"

_oracle = None
_reference = None
u32, u64, vp = C.c_uint32, C.c_uint64, C.c_void_p


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        o = C.CDLL(str(ORACLE_PATH))
        o.rko_f32_to_bf16.restype, o.rko_f32_to_bf16.argtypes = C.c_uint16, [C.c_float]
        o.rko_bf16_to_f32.restype, o.rko_bf16_to_f32.argtypes = C.c_float, [C.c_uint16]
        o.rko_f32_to_e4m3.restype, o.rko_f32_to_e4m3.argtypes = C.c_uint8, [C.c_float]
        o.rko_e4m3_to_f32.restype, o.rko_e4m3_to_f32.argtypes = C.c_float, [C.c_uint8]
        o.rko_query_stage_f16.restype, o.rko_query_stage_f16.argtypes = C.c_float, [C.c_float]
        o.rko_store_chunk.restype = C.c_int
        o.rko_store_chunk.argtypes = [u32, u32, u32, vp, vp, vp, C.POINTER(ChunkParams)]
        o.rko_store_verify.restype = C.c_int
        o.rko_store_verify.argtypes = [u32, u32, u32, u32, vp, vp, vp, vp]
        o.rko_attention_tile.restype = C.c_int
        o.rko_attention_tile.argtypes = [u32, u32, u32, u32, u32, vp, vp, KvLayer, u32, u32, u32, vp, C.c_float,
                                         C.c_int, vp]
        o.rko_attention_verify.restype = C.c_int
        o.rko_attention_verify.argtypes = [u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp]
        o.rko_merge_row.restype = None
        o.rko_merge_row.argtypes = [vp, u64, vp, u64, u32, u32, vp]
        o.rko_tree_compact.restype = C.c_int
        o.rko_tree_compact.argtypes = [u32, u32, u32, vp, C.POINTER(ChunkParams), vp, u32]
        o.rko_copy_page.restype = None
        o.rko_copy_page.argtypes = [u32, u32, u32, u32, u32, u64, u64]
        o.rko_threads.restype = C.c_int
        o.rko_crc32c.restype = C.c_uint32
        o.rko_crc32c.argtypes = [vp, u64, u32]
        o.rko_qkv_prepare.restype = C.c_int
        o.rko_qkv_prepare.argtypes = [u32, u32, u32, u32, u32, vp, vp, vp, C.c_int, vp, vp, C.c_float, vp, vp, vp]
        _oracle = o
    return _oracle


def reference():
    """The reference's own portable code compiled in place, or None where it was not built."""
    global _reference
    if _reference is None and REFERENCE_PATH.exists():
        r = C.CDLL(str(REFERENCE_PATH))
        r.ref_f32_to_bf16.restype, r.ref_f32_to_bf16.argtypes = C.c_uint16, [C.c_float]
        r.ref_bf16_to_f32.restype, r.ref_bf16_to_f32.argtypes = C.c_float, [C.c_uint16]
        r.ref_f32_to_e4m3.restype, r.ref_f32_to_e4m3.argtypes = C.c_uint8, [C.c_float]
        r.ref_e4m3_to_f32.restype, r.ref_e4m3_to_f32.argtypes = C.c_float, [C.c_uint8]
        r.ref_query_stage.restype, r.ref_query_stage.argtypes = C.c_float, [C.c_float]
        r.ref_q8_quantize_page.restype, r.ref_q8_quantize_page.argtypes = C.c_int, [vp, vp, u32, vp]
        r.ref_fp8_quantize_page.restype, r.ref_fp8_quantize_page.argtypes = C.c_int, [vp, vp, u32, vp]
        r.ref_layout.restype, r.ref_layout.argtypes = None, [u32, u32, u32, u32, u64, vp]
        r.ref_kv_offset.restype, r.ref_kv_offset.argtypes = u64, [u32] * 6
        r.ref_key_element.restype, r.ref_key_element.argtypes = u64, [u32] * 4
        r.ref_value_element.restype, r.ref_value_element.argtypes = u64, [u32] * 4
        r.ref_scale_element.restype, r.ref_scale_element.argtypes = u64, [u32] * 2
        r.ref_verify_splits.restype, r.ref_verify_splits.argtypes = u32, [u32, u32]
        r.ref_chunk_validation.restype, r.ref_chunk_validation.argtypes = C.c_char_p, [u32] * 4
        r.ref_verify_plan.restype = C.c_int
        r.ref_verify_plan.argtypes = [u32, u32, u32, u32, u32, u32, vp, C.c_int, C.c_char_p, C.c_size_t, vp]
        r.ref_prefill_plan.restype = C.c_int
        r.ref_prefill_plan.argtypes = [u32, u32, u32, u32, u32, u32, C.c_char_p, C.c_size_t, vp]
        r.ref_workspaces.restype, r.ref_workspaces.argtypes = C.c_int, [u32] * 7 + [vp]
        r.ref_pool_create.restype, r.ref_pool_create.argtypes = vp, [u32, u64, u32, u32, u64]
        r.ref_pool_destroy.restype, r.ref_pool_destroy.argtypes = None, [vp]
        r.ref_pool_set_budget.restype, r.ref_pool_set_budget.argtypes = None, [vp, u64]
        r.ref_pool_acquire.restype, r.ref_pool_acquire.argtypes = C.c_int, [vp, u32, vp]
        r.ref_pool_retain.restype, r.ref_pool_retain.argtypes = C.c_int, [vp, u32, C.c_int]
        r.ref_pool_release.restype, r.ref_pool_release.argtypes = C.c_int, [vp, u32, C.c_int]
        r.ref_pool_reclaim.restype, r.ref_pool_reclaim.argtypes = u64, [vp, C.c_int, u32]
        r.ref_pool_compact.restype, r.ref_pool_compact.argtypes = C.c_int64, [vp, vp, u32, vp]
        r.ref_pool_snapshot.restype, r.ref_pool_snapshot.argtypes = None, [vp, vp]
        if hasattr(r, "ref_cache_create"):  # the request cache facade (a library built before it was added has none)
            i32, i64 = C.c_int, C.c_int64
            r.ref_cache_create.restype, r.ref_cache_create.argtypes = vp, [u32, u64, u32, u32, u64, i32, u32, u32]
            r.ref_cache_destroy.restype, r.ref_cache_destroy.argtypes = None, [vp]
            r.ref_cache_tier_set.restype, r.ref_cache_tier_set.argtypes = None, [vp, u32, i32]
            r.ref_cache_tier_complete.restype, r.ref_cache_tier_complete.argtypes = None, [vp, i32]
            r.ref_cache_begin.restype, r.ref_cache_begin.argtypes = i32, [vp, u64]
            r.ref_cache_end.restype, r.ref_cache_end.argtypes = i32, [vp, u64]
            r.ref_cache_ensure.restype, r.ref_cache_ensure.argtypes = i32, [vp, u64, u64]
            r.ref_cache_page_table.restype, r.ref_cache_page_table.argtypes = i64, [vp, u64, vp, u32, vp, vp]
            r.ref_cache_publish.restype, r.ref_cache_publish.argtypes = i32, [vp, u64, vp, u32, u32, vp, u32]
            r.ref_block_image_identity.restype, r.ref_block_image_identity.argtypes = None, [u64, u32, vp, u32, vp]
            r.ref_cache_block_at.restype, r.ref_cache_block_at.argtypes = u64, [vp, u64, u32]
            r.ref_cache_lookup.restype, r.ref_cache_lookup.argtypes = i32, [vp, vp, u32, i32, i32, u64, vp, vp, vp, u32]
            r.ref_cache_probe_create.restype, r.ref_cache_probe_create.argtypes = vp, [vp, vp, u32, vp, u32]
            r.ref_cache_probe_refresh.restype, r.ref_cache_probe_refresh.argtypes = i32, [vp, vp, vp, u32, vp, u32]
            r.ref_cache_probe_cached_tokens.restype, r.ref_cache_probe_cached_tokens.argtypes = u32, [vp]
            r.ref_cache_probe_destroy.restype, r.ref_cache_probe_destroy.argtypes = None, [vp]
            r.ref_cache_release_lookup.restype, r.ref_cache_release_lookup.argtypes = None, [vp, u64]
            r.ref_cache_restore_status.restype, r.ref_cache_restore_status.argtypes = i32, [vp, u64]
            r.ref_cache_publish_state.restype, r.ref_cache_publish_state.argtypes = i32, [vp, u64, u64, i32]
            r.ref_cache_publish_state_stored.restype, r.ref_cache_publish_state_stored.argtypes = i32, [vp, u64, u64, i32]
            r.ref_cache_use_state.restype, r.ref_cache_use_state.argtypes = i32, [vp, u64, i32]
            r.ref_cache_evict_one.restype, r.ref_cache_evict_one.argtypes = i32, [vp, i32, i32, i32, vp]
            r.ref_cache_reclaim_step.restype, r.ref_cache_reclaim_step.argtypes = i32, [vp, i32, i32, i32, i32, vp]
            r.ref_cache_evict_all.restype, r.ref_cache_evict_all.argtypes = i32, [vp, vp]
            r.ref_cache_reclaim_one_state.restype, r.ref_cache_reclaim_one_state.argtypes = i32, [vp, i32, u64]
            r.ref_cache_block_info.restype, r.ref_cache_block_info.argtypes = i32, [vp, u64, vp]
            r.ref_cache_poll.restype, r.ref_cache_poll.argtypes = i32, [vp]
            r.ref_cache_snapshot.restype, r.ref_cache_snapshot.argtypes = None, [vp, vp]
            if hasattr(r, "ref_cache_adopt"):
                r.ref_cache_adopt.restype, r.ref_cache_adopt.argtypes = i32, [vp, vp, vp, u32, vp, vp, vp, u32, vp]
                r.ref_cache_tier_labels.restype, r.ref_cache_tier_labels.argtypes = i32, [vp, vp, u32]
                r.ref_cache_adopt_labelled.restype, r.ref_cache_adopt_labelled.argtypes = i32, [vp, vp, vp, u32, C.c_char_p, u32, vp]
                r.ref_cache_state_labels.restype, r.ref_cache_state_labels.argtypes = i32, [vp, vp, vp, u32]
        if hasattr(r, "ref_slotfile_write"):  # the persistent slot file
            r.ref_slotfile_write.restype = C.c_int
            r.ref_slotfile_write.argtypes = [C.c_char_p, C.c_char_p, vp, u32, u32, u64, u32, vp, u64, vp]
            r.ref_slotfile_read.restype = C.c_int
            r.ref_slotfile_read.argtypes = [C.c_char_p, C.c_char_p, vp, u32, u32, u64, u32, vp, vp, vp, vp, vp, u64, vp]
        if hasattr(r, "ref_metal_store_verify"):  # the reference's Metal store and compaction kernels run on host threads
            r.ref_metal_store_verify.restype, r.ref_metal_store_verify.argtypes = C.c_int, [u32, vp, vp, vp, vp, u32]
            r.ref_metal_store_chunk.restype, r.ref_metal_store_chunk.argtypes = C.c_int, [u32, vp, vp, vp, vp]
            r.ref_metal_tree_compact.restype, r.ref_metal_tree_compact.argtypes = C.c_int, [u32, vp, vp, vp, vp, u32]
            if hasattr(r, "ref_metal_attention_verify"):
                r.ref_metal_attention_verify.restype = C.c_int
                r.ref_metal_attention_verify.argtypes = [u32, u32, u32, vp, vp, vp, u32, vp, vp, vp, vp, vp, vp]
                if hasattr(r, "ref_metal_qkv_prepare"):
                    r.ref_metal_qkv_prepare.restype = C.c_int
                    r.ref_metal_qkv_prepare.argtypes = [vp, vp, vp, C.c_int, vp, vp, vp, vp, vp, u32, u32]
                r.ref_metal_attention_prefill.restype = C.c_int
                r.ref_metal_attention_prefill.argtypes = [u32, vp, vp, vp, vp, vp, vp]
        _reference = r
    return _reference


def ptr(array: np.ndarray) -> int:
    return array.ctypes.data
