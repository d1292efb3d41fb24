"""Host-side mirror of the KV ABI: formats, parameter blocks and byte accounting.

The numbers restate include/richkv_abi.h (which restates the reference's
runtime/metal/abi/*.h and runtime/ops/PagedKv.hpp:125-232); the parameter
dtypes are numpy views of the same 24/32/36-byte blocks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

PAGE_TOKENS = 32
VERIFY_ROWS = 8
TREE_NODES = 16
MAX_CONTEXT_TOKENS = 262144
MAX_PHYSICAL_TOKENS = MAX_CONTEXT_TOKENS + TREE_NODES - 1
PREFILL_TOKEN_BUDGET = 2048
VERIFY_CHUNK_STRIDE = PAGE_TOKENS
PREFILL_TILE_ROWS = 8
PREFILL_MAX_SPLITS = 32
VERIFY_MAX_SPLITS = 128
VERIFY_SPLITS = 32
VERIFY_PAGES_PER_SPLIT = 16
PAGE_INDEX_BITS = 14
PAGE_INDEX_MASK = (1 << PAGE_INDEX_BITS) - 1

INT8, BF16, INT4, FP8E4M3 = 1, 2, 3, 4
FORMAT_NAMES = {INT8: "int8", BF16: "bf16", INT4: "int4", FP8E4M3: "fp8e4m3"}
FORMAT_TAGS = {INT8: "q8", BF16: "bf16", INT4: "int4", FP8E4M3: "fp8"}

KV_LAYER = np.dtype([("extent_pages", "<u4"), ("offset", "<u4")])
CHUNK_PARAMS = np.dtype([("committed_tokens", "<u4"), ("chunk_tokens", "<u4"), ("chunk_stride", "<u4"),
                         ("page_table_entries", "<u4"), ("kv", KV_LAYER)])
PREFILL_PARAMS = np.dtype([("committed_tokens", "<u4"), ("rows", "<u4"), ("chunk_stride", "<u4"),
                           ("page_table_entries", "<u4"), ("kv", KV_LAYER), ("split_count", "<u4"),
                           ("score_scale", "<f4")])
VERIFY_PARAMS = np.dtype([("committed_tokens", "<u4"), ("page_table_entries", "<u4"), ("kv", KV_LAYER),
                          ("split_count", "<u4"), ("slot_splits", "<u4"), ("active_rows", "<u4"),
                          ("row_capacity", "<u4"), ("score_scale", "<f4")])
PAGE_COPY = np.dtype([("from", "<u4"), ("to", "<u4")])
assert KV_LAYER.itemsize == 8 and CHUNK_PARAMS.itemsize == 24
assert PREFILL_PARAMS.itemsize == 32 and VERIFY_PARAMS.itemsize == 36 and PAGE_COPY.itemsize == 8

EXTENT_REGION_ALIGNMENT = 64 * 1024
ALLOCATION_EXTENT_TARGET = 128 * 1024 * 1024


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass(frozen=True)
class Layout:
    """kv::Layout (runtime/ops/PagedKv.hpp:125-232)."""

    attention_layers: int
    kv_heads: int
    head_dimension: int
    format: int = INT8
    score_scale: float = 0.0

    def valid(self) -> bool:
        return bool(self.attention_layers and self.kv_heads and self.head_dimension and self.format in FORMAT_NAMES)

    def quantized(self) -> bool:
        return self.format != BF16

    def elements_per_layer_page(self) -> int:
        return PAGE_TOKENS * self.kv_heads * self.head_dimension

    def data_bytes_per_layer_page(self) -> int:
        elements = self.elements_per_layer_page()
        if self.format == BF16:
            return elements * 2
        if self.format == INT4:
            return elements // 2
        return elements

    def scale_bytes_per_layer_page(self) -> int:
        return PAGE_TOKENS * self.kv_heads * 4 if self.quantized() else 0

    def bytes_per_layer_page(self) -> int:
        return 2 * (self.data_bytes_per_layer_page() + self.scale_bytes_per_layer_page())

    def bytes_per_model_page(self) -> int:
        return self.attention_layers * self.bytes_per_layer_page()

    def bytes_per_token_layer(self) -> int:
        return self.bytes_per_layer_page() // PAGE_TOKENS

    @staticmethod
    def _pages_for_aligned_region(bytes_per_page: int) -> int:
        return EXTENT_REGION_ALIGNMENT // math.gcd(EXTENT_REGION_ALIGNMENT, bytes_per_page) if bytes_per_page else 0

    def extent_alignment_pages(self) -> int:
        data = self._pages_for_aligned_region(self.data_bytes_per_layer_page())
        if self.format == BF16:
            return data
        return math.lcm(data, self._pages_for_aligned_region(self.scale_bytes_per_layer_page()))

    def minimum_extent_pages(self) -> int:
        unit = self.extent_alignment_pages() * self.bytes_per_model_page()
        if not unit:
            return 0
        units = max(1, (ALLOCATION_EXTENT_TARGET // 2 + unit - 1) // unit)
        return units * self.extent_alignment_pages()

    def maximum_extent_pages(self) -> int:
        unit = self.extent_alignment_pages() * self.bytes_per_model_page()
        if not unit:
            return 0
        units = ALLOCATION_EXTENT_TARGET * 3 // 2 // unit
        return max(units * self.extent_alignment_pages(), self.minimum_extent_pages())

    def extent_pages_for(self, pages: int) -> int:
        """The extent size of a pool of `pages` pages: fewest pages left over, nearest the target on a tie."""
        step, smallest = self.extent_alignment_pages(), self.minimum_extent_pages()
        if not smallest or pages < smallest:
            return 0
        largest = min(self.maximum_extent_pages(), pages)
        best = best_left = best_distance = 0
        extent = smallest
        while extent <= largest:
            distance = abs(extent * self.bytes_per_model_page() - ALLOCATION_EXTENT_TARGET)
            left = pages % extent
            if not best or left < best_left or (left == best_left and distance < best_distance):
                best, best_left, best_distance = extent, left, distance
            extent += step
        return best

    def layer_offset(self, extent_pages: int, layer: int, tensor: int = 0, index: int = 0) -> int:
        data, scale = self.data_bytes_per_layer_page(), self.scale_bytes_per_layer_page()
        region = layer * extent_pages * 2 * (data + scale)
        before = (tensor + 1) // 2 * data + tensor // 2 * scale
        return region + extent_pages * before + index * (scale if tensor % 2 else data)


def verify_attention_splits(committed_tokens: int, rows: int = VERIFY_ROWS) -> int:
    """kv::verifyAttentionSplits (runtime/ops/PagedAttention.hpp:54-63)."""
    pages = pages_for(committed_tokens + rows)
    scaled = (pages + VERIFY_PAGES_PER_SPLIT - 1) // VERIFY_PAGES_PER_SPLIT
    return min(max(VERIFY_SPLITS, scaled), VERIFY_MAX_SPLITS)


def prefill_splits(tiles: int) -> int:
    """prefillSplits (runtime/ops/PagedAttention.cpp:23-26)."""
    return min(max(PREFILL_MAX_SPLITS // tiles, 1), PREFILL_MAX_SPLITS)
