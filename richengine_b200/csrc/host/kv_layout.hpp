// kv_layout.hpp — host-side KV geometry and the storage interface the pool drives.
//
// Mirrors the reference's operator-layer types so host code written against them
// ports by namespace: kv::Format / kv::Layout / kv::PageCopy / kv::ExtentStorage
// (runtime/ops/PagedKv.hpp:16-232) and metal::AllocationFailure / AllocationResult
// (runtime/metal/MetalBackend.hpp:18-33). Byte arithmetic comes from the shared ABI
// header, so host and kernels cannot disagree.
#pragma once

#include "../../../include/richkv_abi.h"

#include <algorithm>
#include <cstdint>
#include <numeric>
#include <span>
#include <string_view>

namespace rkb {

enum class AllocationFailure : uint8_t { None, EngineBudget, HostPressure, DriverRejected };

struct AllocationResult final {
  AllocationFailure failure = AllocationFailure::None;
  AllocationResult() noexcept = default;
  AllocationResult(AllocationFailure reason) noexcept : failure(reason) {}
  explicit operator bool() const noexcept { return failure == AllocationFailure::None; }
};

namespace kv {

enum class Format : uint32_t { Int8 = RK_FORMAT_INT8, BFloat16 = RK_FORMAT_BF16, Int4 = RK_FORMAT_INT4, Float8E4M3 = RK_FORMAT_FP8E4M3 };

constexpr bool validFormat(Format f) noexcept { return rk_format_valid(static_cast<uint32_t>(f)) != 0; }
constexpr std::string_view formatName(Format f) noexcept {
  switch (f) {
  case Format::Int8: return "int8";
  case Format::BFloat16: return "bf16";
  case Format::Int4: return "int4";
  case Format::Float8E4M3: return "fp8e4m3";
  }
  return "invalid";
}

inline constexpr uint32_t kPageTokens = RK_PAGE_TOKENS;
inline constexpr uint32_t kMaximumPhysicalTokens = RK_MAX_PHYSICAL_TOKENS;
inline constexpr uint64_t kExtentRegionAlignmentBytes = 64 * 1024;
inline constexpr uint64_t kAllocationExtentTargetBytes = 128ull * 1024 * 1024;

struct PageCopy final {
  uint32_t from = 0;
  uint32_t to = 0;
};

// Physical KV geometry of a pool (PagedKv.hpp:125-232).
struct Layout final {
  uint32_t attentionLayers = 0, kvHeads = 0, headDimension = 0;
  Format format = Format::Int8;
  float scoreScale = 0.0f;

  constexpr bool valid() const noexcept { return attentionLayers && kvHeads && headDimension && validFormat(format); }
  constexpr bool quantized() const noexcept { return format != Format::BFloat16; }
  constexpr uint64_t dataBytesPerLayerPage() const noexcept { return rk_data_bytes(uint32_t(format), kvHeads, headDimension); }
  constexpr uint64_t scaleBytesPerLayerPage() const noexcept { return rk_scale_bytes(uint32_t(format), kvHeads); }
  constexpr uint64_t bytesPerLayerPage() const noexcept { return 2 * (dataBytesPerLayerPage() + scaleBytesPerLayerPage()); }
  constexpr uint64_t bytesPerModelPage() const noexcept { return attentionLayers * bytesPerLayerPage(); }

  static constexpr uint64_t pagesForAlignedRegion(uint64_t bytes) noexcept {
    return bytes ? kExtentRegionAlignmentBytes / std::gcd(kExtentRegionAlignmentBytes, bytes) : 0;
  }
  constexpr uint32_t extentAlignmentPages() const noexcept {
    const uint64_t data = pagesForAlignedRegion(dataBytesPerLayerPage());
    if (!quantized()) return uint32_t(data);
    return uint32_t(std::lcm(data, pagesForAlignedRegion(scaleBytesPerLayerPage())));
  }
  constexpr uint32_t minimumExtentPages() const noexcept {
    const uint64_t unit = uint64_t(extentAlignmentPages()) * bytesPerModelPage();
    if (!unit) return 0;
    return uint32_t(std::max<uint64_t>(1, (kAllocationExtentTargetBytes / 2 + unit - 1) / unit) * extentAlignmentPages());
  }
  constexpr uint32_t maximumExtentPages() const noexcept {
    const uint64_t unit = uint64_t(extentAlignmentPages()) * bytesPerModelPage();
    if (!unit) return 0;
    return std::max(uint32_t(kAllocationExtentTargetBytes * 3 / 2 / unit * extentAlignmentPages()), minimumExtentPages());
  }
  // The extent size of a pool of `pages` pages: fewest pages left over, nearest the target on a tie.
  constexpr uint32_t extentPagesFor(uint64_t pages) const noexcept {
    const uint64_t step = extentAlignmentPages(), smallest = minimumExtentPages();
    if (!smallest || pages < smallest) return 0;
    const uint64_t largest = std::min<uint64_t>(maximumExtentPages(), pages);
    uint64_t best = 0, bestLeft = 0, bestDistance = 0;
    for (uint64_t extent = smallest; extent <= largest; extent += step) {
      const uint64_t bytes = extent * bytesPerModelPage();
      const uint64_t distance = bytes > kAllocationExtentTargetBytes ? bytes - kAllocationExtentTargetBytes
                                                                     : kAllocationExtentTargetBytes - bytes;
      if (!best || pages % extent < bestLeft || (pages % extent == bestLeft && distance < bestDistance)) {
        best = extent; bestLeft = pages % extent; bestDistance = distance;
      }
    }
    return uint32_t(best);
  }
  bool operator==(const Layout &) const = default;
};

// The memory of a page pool: extents of extentPages() pages that only the pool
// allocates and releases (PagedKv.hpp:56-76).
class ExtentStorage {
public:
  virtual ~ExtentStorage() = default;
  virtual uint32_t pageCount() const noexcept = 0;
  virtual uint64_t bytesPerPage() const noexcept = 0;
  virtual uint32_t extentPages() const noexcept = 0;
  // Granted, or the refusal's cause with nothing allocated; std::logic_error for an allocated extent.
  virtual AllocationResult allocateExtent(uint32_t extent) = 0;
  // std::logic_error, changing nothing, for an unallocated extent.
  virtual void releaseExtent(uint32_t extent) = 0;
  // Copies each page's content onto its destination; std::logic_error, copying nothing, for a page
  // of an unallocated extent.
  virtual void copyPages(std::span<const PageCopy> copies) = 0;
};

} // namespace kv
} // namespace rkb
