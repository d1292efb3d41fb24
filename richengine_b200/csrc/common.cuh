// common.cuh — device helpers shared by the paged-KV kernels.
#pragma once

#include "../../include/richkv.h"

#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rk {

constexpr uint32_t kPageTokens = RK_PAGE_TOKENS;

// Status codes every C entry point returns (include/richkv.h).
constexpr int kOk = 0;
constexpr int kInvalid = -1;     // host-side contract violation, nothing launched
constexpr int kCudaError = -2;   // a CUDA call failed; rk_last_error() has the text
constexpr int kUnsupported = -3; // geometry or format without a kernel
constexpr int kRefused = -4;     // capacity refusal (allocator, tier)
constexpr int kTimeout = -5;     // a bounded device wait ran out

void set_error(const char *text);
int cuda_status(cudaError_t error, const char *what);

// Pages of one host-tier batch, carried in a kernel's arguments: nothing is copied or allocated per transfer.
constexpr uint32_t kTierBatch = 16;
struct PageBatch {
  rk_page_entry entry[kTierBatch]; // the pages' table entries
  uint8_t *slot[kTierBatch];       // their packed device slots
  uint32_t *publish[kTierBatch];   // seal only: the host-visible word each checksum is stored to
};

// Host-side description of a seal (pack + checksum in one pass): the pages' table entries (device memory) and the
// pool's span geometry. A seal for the host tier carries its pages in `batch` instead (`entries` null): every payload
// has its own destination slot and a host-visible word its finished checksum is stored to; `arrivals` and the
// accumulators are device words, one per payload, that are zero between launches (the last part of a payload to
// finish stores the checksum and clears both), so one launch replaces a copy of the entries, a clear, the kernel and
// the copies of the checksums.
struct GatherSource {
  const rk_page_entry *entries;
  uint32_t layers, extent_pages, data_bytes, scale_bytes;
  const PageBatch *batch = nullptr;
  uint32_t *arrivals = nullptr;
};

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits) { return __uint_as_float(bits << 16); }

// Round-to-nearest-even fp32 -> bf16 bits; quiet NaNs stay NaN.
__device__ __forceinline__ uint16_t float_to_bf16_bits(float value) {
  uint32_t bits = __float_as_uint(value);
  if ((bits & 0x7f800000u) == 0x7f800000u) {
    uint16_t upper = uint16_t(bits >> 16);
    if ((bits & 0x007fffffu) && !(upper & 0x007fu)) upper |= 1;
    return upper;
  }
  return uint16_t((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Pointers to one KV head's slab of each tensor of one page in one layer
// (runtime/metal/kernels/common/kv_extent.h:53-108).
struct PageSlabs {
  uint8_t *keys;
  uint8_t *values;
  float *key_scales;
  float *value_scales;
};

template <uint32_t Format, uint32_t KvHeads, uint32_t HeadDim> struct PageGeometry {
  static constexpr bool kQuantized = Format != RK_FORMAT_BF16;
  static constexpr uint32_t kElementBits = Format == RK_FORMAT_BF16 ? 16 : (Format == RK_FORMAT_INT4 ? 4 : 8);
  static constexpr uint32_t kDataBytes = kPageTokens * KvHeads * HeadDim * kElementBits / 8;
  static constexpr uint32_t kScaleBytes = kQuantized ? kPageTokens * KvHeads * 4 : 0;
  static constexpr uint32_t kHeadDataBytes = kDataBytes / KvHeads;
  static constexpr uint32_t kRowBytes = HeadDim * kElementBits / 8; // one token-major row

  __device__ __forceinline__ static PageSlabs slabs(rk_page_entry entry, rk_kv_layer layer, uint32_t head) {
    const uint32_t index = rk_entry_index(entry);
    uint8_t *region = reinterpret_cast<uint8_t *>(rk_entry_extent(entry)) + layer.offset;
    const uint64_t pages = layer.extent_pages;
    PageSlabs s;
    s.keys = region + uint64_t(index) * kDataBytes + head * kHeadDataBytes;
    s.values = region + pages * (uint64_t(kDataBytes) + kScaleBytes) + uint64_t(index) * kDataBytes +
               head * kHeadDataBytes;
    if (kQuantized) {
      s.key_scales = reinterpret_cast<float *>(region + pages * kDataBytes + uint64_t(index) * kScaleBytes) +
                     head * kPageTokens;
      s.value_scales = reinterpret_cast<float *>(region + pages * (2ull * kDataBytes + kScaleBytes) +
                                                 uint64_t(index) * kScaleBytes) +
                       head * kPageTokens;
    } else {
      s.key_scales = nullptr;
      s.value_scales = nullptr;
    }
    return s;
  }
};

// ---- the quantiser shared by the stores (store.cu, qkv_prepare.cu) ----
template <uint32_t Format> struct Quantizer;
template <> struct Quantizer<RK_FORMAT_INT8> { static constexpr float kRange = 127.0f; };
template <> struct Quantizer<RK_FORMAT_INT4> { static constexpr float kRange = 7.0f; };
template <> struct Quantizer<RK_FORMAT_FP8E4M3> { static constexpr float kRange = 448.0f; };

// The stored code of one element: an int8/int4 two's-complement code or an
// e4m3 byte. (x*range)/amax is two IEEE round-to-nearest operations; no
// reciprocal and no fused multiply-add may replace them.
template <uint32_t Format> __device__ __forceinline__ uint32_t encode(float value, float amax) {
  if (amax == 0.0f) return 0u;
  const float scaled = __fdiv_rn(__fmul_rn(value, Quantizer<Format>::kRange), amax);
  if (Format == RK_FORMAT_FP8E4M3)
    return uint32_t(__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3));
  const int limit = int(Quantizer<Format>::kRange);
  const int q = max(-limit, min(limit, __float2int_rn(scaled)));
  return uint32_t(q) & (Format == RK_FORMAT_INT4 ? 0xFu : 0xFFu);
}

// One stored element's code as a float, before its scale
// (K token-major for all formats; V token-major only for INT4).
template <uint32_t Format>
__device__ __forceinline__ float decode_element(const uint8_t *slab, uint32_t element) {
  if (Format == RK_FORMAT_INT8) return float(reinterpret_cast<const int8_t *>(slab)[element]);
  if (Format == RK_FORMAT_INT4) {
    const int code = (slab[element >> 1] >> ((element & 1u) * 4u)) & 0xF;
    return float(code - ((code & 8) ? 16 : 0));
  }
  if (Format == RK_FORMAT_FP8E4M3) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(slab[element], __NV_E4M3);
    return __half2float(__half(h));
  }
  return bf16_bits_to_float(reinterpret_cast<const uint16_t *>(slab)[element]);
}

} // namespace rk
