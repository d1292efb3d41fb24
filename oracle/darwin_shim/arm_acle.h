/* Stands in for <arm_acle.h> when the reference's portable sources are compiled on x86-64 Linux for the test-only
 * checker: its two CRC-32C intrinsics, computed bit by bit (polynomial 0x82F63B78, reflected), so that the reference's
 * own Crc32c.hpp runs unchanged. */
#pragma once
#include <stdint.h>
static inline uint32_t rk_shim_crc32c_byte(uint32_t state, uint8_t byte) {
  state ^= byte;
  for (int bit = 0; bit < 8; ++bit) state = (state >> 1) ^ (0x82F63B78u & (0u - (state & 1u)));
  return state;
}
static inline uint32_t __crc32cb(uint32_t state, uint8_t value) { return rk_shim_crc32c_byte(state, value); }
static inline uint32_t __crc32cd(uint32_t state, uint64_t value) {
  for (int byte = 0; byte < 8; ++byte) state = rk_shim_crc32c_byte(state, (uint8_t)(value >> (8 * byte)));
  return state;
}
