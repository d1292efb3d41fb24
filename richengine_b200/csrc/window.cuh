// window.cuh — the device address window of a pool and its TMA tensor maps.
//
// Every extent of a pool is mapped inside one virtual address range (rk_storage_window), so a tensor
// map of 128-byte rows covers every page whatever the format: one head's K (or V) slab of a page is 32
// (int4), 64 (int8, fp8) or 128 (bf16) consecutive rows, all four heads of an int4 page 128. The maps
// over the same rows differ only in the box.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace rk {

struct Window {
  uint64_t base = 0, bytes = 0;
  CUtensorMap int4_map;      // box = 128 rows: all heads of an int4 page (also one head's bf16 slab)
  CUtensorMap int4_head_map; // box = 32 rows: one head's int4 slab
  CUtensorMap byte_head_map; // box = 64 rows: one head's int8 / fp8 slab
};

int encode_window_map(CUtensorMap *map, uint64_t base, uint64_t rows, uint32_t box_rows);

} // namespace rk
