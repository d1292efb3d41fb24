// window.cuh — the device address window of a pool and its TMA tensor maps.
//
// Every extent of a pool is mapped inside one virtual address range (rk_storage_window), so a single
// tensor map of 128-byte rows covers every int4 page: a page's K (or V) data of all four heads is 128
// consecutive rows, one head's slab 32 of them. Two maps over the same rows differ only in the box:
// 128 rows (the decode kernel copies all heads of a page at once) and 32 rows (one head's slab).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace rk {

struct Window {
  uint64_t base = 0, bytes = 0;
  CUtensorMap int4_map;      // box = 128 rows: all heads of a page
  CUtensorMap int4_head_map; // box = 32 rows: one head's slab
};

int encode_window_map(CUtensorMap *map, uint64_t base, uint64_t rows, uint32_t box_rows);

} // namespace rk
