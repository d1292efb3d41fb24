"""kv::PageStorage for CUDA (runtime/ops/PageStorage.hpp:27-102) over the C ABI.

Extents are physical allocations mapped into one reserved device address
window; a page is reached through its 64-bit table entry. Only the pool
allocates and releases extents (runtime/engine/cache/KvPool.hpp:64-74).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib
from .abi import Layout


class AllocationRefused(RuntimeError):
    """The budget or the driver refused to grow the pool by an extent."""


class PageStorage:
    def __init__(self, layout: Layout, page_count: int, extent_pages: int):
        if not layout.valid():
            raise ValueError("KV page storage layout is invalid")
        self._lib = lib.load()
        self.layout = layout
        self._handle = self._lib.rk_storage_create(layout.format, layout.attention_layers, layout.kv_heads,
                                                   layout.head_dimension, page_count, extent_pages)
        if not self._handle:
            raise ValueError(self._lib.rk_last_error().decode())
        self.page_count = page_count
        self.extent_pages = extent_pages

    def close(self) -> None:
        if self._handle:
            self._lib.rk_storage_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._handle

    def bytes_per_page(self) -> int:
        return self._lib.rk_storage_bytes_per_page(self._handle)

    def extent_bytes(self) -> int:
        return self._lib.rk_storage_extent_bytes(self._handle)

    def actual_allocated_bytes(self) -> int:
        return self._lib.rk_storage_allocated_bytes(self._handle)

    def is_allocated(self, page: int) -> bool:
        return bool(self._lib.rk_storage_is_allocated(self._handle, page))

    def set_budget(self, bytes_: int) -> None:
        self._lib.rk_storage_set_budget(self._handle, bytes_)

    def allocate_extent(self, extent: int) -> bool:
        """True when granted, False when refused (budget or driver); raises on misuse."""
        status = self._lib.rk_storage_allocate_extent(self._handle, extent)
        if status == lib.REFUSED:
            return False
        if status == lib.INVALID:
            raise RuntimeError(self._lib.rk_last_error().decode())
        lib.check(status, "allocate_extent")
        return True

    def release_extent(self, extent: int) -> None:
        status = self._lib.rk_storage_release_extent(self._handle, extent)
        if status == lib.INVALID:
            raise RuntimeError(self._lib.rk_last_error().decode())
        lib.check(status, "release_extent")

    def window(self) -> tuple[int, int]:
        base, size = C.c_uint64(), C.c_uint64()
        self._lib.rk_storage_window(self._handle, C.byref(base), C.byref(size))
        return base.value, size.value

    def layers(self) -> list[lib.KvLayer]:
        count = self.layout.attention_layers
        out = (lib.KvLayer * count)()
        self._lib.rk_storage_layers(self._handle, out, count)
        return [lib.KvLayer(x.extent_pages, x.offset) for x in out]

    def entry(self, page: int) -> int:
        value = self._lib.rk_storage_entry(self._handle, page)
        if not value:
            raise RuntimeError(f"KV page {page} is in an extent that is not allocated")
        return value

    def write_entries(self, pages, first: int, table, stream: int = 0) -> None:
        """pages: sequence of page ids; table: a torch int64/uint64 device tensor."""
        ids = np.ascontiguousarray(pages, dtype=np.uint32)
        status = self._lib.rk_storage_write_entries(self._handle, ids.ctypes.data, len(ids), first, table.data_ptr(),
                                                    table.numel(), stream)
        if status == lib.INVALID:
            raise RuntimeError(self._lib.rk_last_error().decode())
        lib.check(status, "write_entries")

    def copy_pages(self, copies, stream: int = 0) -> None:
        pairs = np.ascontiguousarray(copies, dtype=np.uint32).reshape(-1, 2)
        status = self._lib.rk_storage_copy_pages(self._handle, pairs.ctypes.data, len(pairs), stream)
        if status == lib.INVALID:
            raise RuntimeError(self._lib.rk_last_error().decode())
        lib.check(status, "copy_pages")

    def read_extent(self, extent: int) -> np.ndarray:
        out = np.empty(self.extent_bytes(), dtype=np.uint8)
        lib.check(self._lib.rk_storage_read_extent(self._handle, extent, 0, out.ctypes.data, out.nbytes), "read_extent")
        return out

    def write_extent(self, extent: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data, dtype=np.uint8)
        lib.check(self._lib.rk_storage_write_extent(self._handle, extent, 0, data.ctypes.data, data.nbytes), "write_extent")
