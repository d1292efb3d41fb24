"""Test scenarios: a host-memory mirror of the page pool for the CPU checker and,
where a GPU exists, the same pool on the device with identical page ids.

HostPool follows the reference's CPU-visible test extents
(dev/tuning/HostKvExtents.hpp:27-186): production addressing over host
buffers, >= 3 extents, pages handed out from a seeded shuffle.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from richengine_b200 import abi, lib
from richengine_b200.abi import Layout

import oracle as oracle_module

GEOMETRY_27B = dict(kv_heads=4, head_dimension=256)
QUERY_HEADS = 24


# ---- bf16 helpers ------------------------------------------------------------------
def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class HostPool:
    """Host extents addressed exactly like device extents."""

    def __init__(self, layout: Layout, extent_pages: int, extents: int):
        self.layout, self.extent_pages, self.extents = layout, extent_pages, extents
        self.extent_bytes = extent_pages * layout.bytes_per_model_page()
        self._raw = [np.zeros(self.extent_bytes + 16384, dtype=np.uint8) for _ in range(extents)]
        self.bytes = []
        for raw in self._raw:
            shift = (-raw.ctypes.data) % 16384
            self.bytes.append(raw[shift:shift + self.extent_bytes])
        self.page_count = extent_pages * extents

    def address(self, extent: int) -> int:
        return self.bytes[extent].ctypes.data

    def entry(self, page: int) -> int:
        extent, index = divmod(page, self.extent_pages)
        return self.address(extent) | index

    def layer(self, index: int) -> lib.KvLayer:
        return lib.KvLayer(self.extent_pages, self.layout.layer_offset(self.extent_pages, index))

    def table(self, pages) -> np.ndarray:
        return np.array([self.entry(p) for p in pages], dtype=np.uint64)

    def tensor_view(self, page: int, layer: int, tensor: int) -> np.ndarray:
        extent, index = divmod(page, self.extent_pages)
        offset = self.layout.layer_offset(self.extent_pages, layer, tensor, index)
        size = self.layout.scale_bytes_per_layer_page() if tensor % 2 else self.layout.data_bytes_per_layer_page()
        return self.bytes[extent][offset:offset + size]


class Scenario:
    """`lanes` sequences with their page lists over a pool, mirrored on host (and device)."""

    def __init__(self, layout: Layout, contexts, extra_tokens: int = 0, seed: int = 7, device: bool = False,
                 extent_pages: int | None = None, min_extents: int = 3):
        self.layout = layout
        self.contexts = [int(c) for c in contexts]
        self.lanes = len(self.contexts)
        self.rng = np.random.default_rng(seed)
        need = sum(abi.pages_for(c + extra_tokens) for c in self.contexts) + 8  # spare pages for copies
        self.extent_pages = extent_pages or layout.extent_alignment_pages()
        extents = max(min_extents, (need + self.extent_pages - 1) // self.extent_pages)
        self.host = HostPool(layout, self.extent_pages, extents)
        order = self.rng.permutation(self.host.page_count)
        self.pages, cursor = [], 0
        for c in self.contexts:
            count = abi.pages_for(c + extra_tokens)
            self.pages.append([int(p) for p in order[cursor:cursor + count]])
            cursor += count
        self.spare_pages = [int(p) for p in order[cursor:]]
        self.host_tables = [self.host.table(p) for p in self.pages]
        self.storage = None
        self.device_tables = None
        if device:
            self.attach_device()

    # -- device mirror ----------------------------------------------------------------
    def attach_device(self):
        import torch
        from richengine_b200.storage import PageStorage
        self.storage = PageStorage(self.layout, self.host.page_count, self.extent_pages)
        for extent in range(self.host.extents):
            assert self.storage.allocate_extent(extent)
        self.device_tables = []
        for pages in self.pages:
            table = torch.zeros(max(len(pages), 1), dtype=torch.int64, device="cuda")
            self.storage.write_entries(pages, 0, table)
            self.device_tables.append(table)
        from richengine_b200 import ops
        self.table_pointers = ops.table_pointer_array(self.device_tables)
        torch.cuda.synchronize()

    def upload(self):
        """Host extents -> device extents."""
        for extent in range(self.host.extents):
            self.storage.write_extent(extent, self.host.bytes[extent])

    def download(self):
        return [self.storage.read_extent(e) for e in range(self.host.extents)]

    def host_table_pointers(self):
        holder = (C.c_void_p * self.lanes)(*[t.ctypes.data for t in self.host_tables])
        return holder

    def close(self):
        if self.storage is not None:
            self.storage.close()
            self.storage = None


def fill_history_with_store(scenario: Scenario, layer_index: int, seed: int = 11, chunk: int = 256):
    """Fills every lane's committed history on the HOST mirror through the checker's store
    (bf16 synthetic rows -> quantized pages), chunk by chunk."""
    o = oracle_module.oracle()
    layout = scenario.layout
    H, D = layout.kv_heads, layout.head_dimension
    rng = np.random.default_rng(seed)
    layer = scenario.host.layer(layer_index)
    for lane, context in enumerate(scenario.contexts):
        done = 0
        while done < context:
            rows = min(chunk, context - done)
            stride = (rows + 31) // 32 * 32
            k = np.zeros((H, stride, D), dtype=np.uint16)
            v = np.zeros((H, D, stride), dtype=np.uint16)
            k[:, :rows, :] = _rows_with_outliers(rng, H, rows, D, 101)
            v[:, :, :rows] = _rows_with_outliers(rng, H, rows, D, 202).transpose(0, 2, 1)
            params = lib.ChunkParams(done, rows, stride, len(scenario.pages[lane]), layer)
            status = o.rko_store_chunk(layout.format, H, D, k.ctypes.data, v.ctypes.data,
                                       scenario.host_tables[lane].ctypes.data, C.byref(params))
            assert status == 0
            done += rows


def _rows_with_outliers(rng, heads: int, rows: int, dim: int, channel_seed: int) -> np.ndarray:
    """bf16 bits [heads][rows][dim]: N(0,1) with 4 seeded outlier channels per head x20."""
    x = rng.standard_normal((heads, rows, dim), dtype=np.float32)
    channel_rng = np.random.default_rng(channel_seed)
    for head in range(heads):
        x[head][:, channel_rng.choice(dim, size=4, replace=False)] *= 20.0
    return f32_to_bf16(x)


def make_queries(rng, lanes: int, layout: Layout, query_heads: int = QUERY_HEADS, stride: int = 32) -> np.ndarray:
    """bf16 bits [lane][kv_head][stride][group][D] ~ N(0,1) with outlier channels."""
    H, D = layout.kv_heads, layout.head_dimension
    group = query_heads // H
    x = rng.standard_normal((lanes, H, stride, group, D), dtype=np.float32)
    channel_rng = np.random.default_rng(303)
    for head in range(H):
        x[:, head][..., channel_rng.choice(D, size=4, replace=False)] *= 20.0
    return f32_to_bf16(x)


def make_staging(rng, lanes: int, layout: Layout, stride: int = 32):
    """Chunk staging for a verify/decode store: K [lane][H][stride][D], V [lane][H][D][stride]."""
    H, D = layout.kv_heads, layout.head_dimension
    k = np.stack([_rows_with_outliers(rng, H, stride, D, 101) for _ in range(lanes)])
    v = np.stack([_rows_with_outliers(rng, H, stride, D, 202).transpose(0, 2, 1) for _ in range(lanes)])
    return np.ascontiguousarray(k), np.ascontiguousarray(v)
