// storage_adapters.hpp — kv::ExtentStorage over the CUDA extent storage of the C ABI, and a
// memory-less storage for host-only use (tests, CPU ranks).
#pragma once

#include "../../../include/richkv.h"
#include "kv_layout.hpp"

#include <stdexcept>
#include <string>
#include <vector>

namespace rkb::kv {

// Adapter the pool drives on a GPU: rk_storage_* (capi.cu). Copies are ordered on `stream`.
class DeviceExtentStorage final : public ExtentStorage {
public:
  explicit DeviceExtentStorage(void *storage, void *stream = nullptr) : storage_(storage), stream_(stream) {
    if (!storage_) throw std::invalid_argument("null KV storage handle");
  }
  uint32_t pageCount() const noexcept override { return rk_storage_page_count(storage_); }
  uint64_t bytesPerPage() const noexcept override { return rk_storage_bytes_per_page(storage_); }
  uint32_t extentPages() const noexcept override { return rk_storage_extent_pages(storage_); }
  AllocationResult allocateExtent(uint32_t extent) override {
    const int status = rk_storage_allocate_extent(storage_, extent);
    if (status == RK_OK) return {};
    if (status == RK_ERR_REFUSED) return AllocationFailure::EngineBudget;
    if (status == RK_ERR_INVALID) throw std::logic_error(rk_last_error());
    return AllocationFailure::DriverRejected;
  }
  void releaseExtent(uint32_t extent) override {
    if (rk_storage_release_extent(storage_, extent) != RK_OK) throw std::logic_error(rk_last_error());
  }
  void copyPages(std::span<const PageCopy> copies) override {
    static_assert(sizeof(PageCopy) == sizeof(rk_page_copy));
    if (rk_storage_copy_pages(storage_, reinterpret_cast<const rk_page_copy *>(copies.data()), uint32_t(copies.size()), stream_) != RK_OK)
      throw std::logic_error(rk_last_error());
  }
  void *handle() const noexcept { return storage_; }

private:
  void *storage_;
  void *stream_;
};

// No memory: a page budget decides growth, a copy log records moves, and every page carries one
// 64-bit content tag that copies move (the shape of the reference's test storage,
// dev/tests/engine/TestKvPool.hpp:27-113).
class BudgetExtentStorage final : public ExtentStorage {
public:
  BudgetExtentStorage(uint32_t pages, uint64_t bytesPerPage, uint32_t extentPages)
      : content(pages), pages_(pages), bytes_(bytesPerPage), extent_(extentPages), allocated_(extentPages ? pages / extentPages : 0) {}
  uint32_t pageCount() const noexcept override { return pages_; }
  uint64_t bytesPerPage() const noexcept override { return bytes_; }
  uint32_t extentPages() const noexcept override { return extent_; }
  AllocationResult allocateExtent(uint32_t extent) override {
    if (allocated_.at(extent)) throw std::logic_error("KV extent is already allocated");
    uint64_t held = 0;
    for (bool a : allocated_) held += a;
    if ((held + 1) * extent_ > budgetPages) return AllocationFailure::EngineBudget;
    allocated_[extent] = true;
    return {};
  }
  void releaseExtent(uint32_t extent) override {
    if (!allocated_.at(extent)) throw std::logic_error("KV extent is not allocated");
    allocated_[extent] = false;
  }
  void copyPages(std::span<const PageCopy> copies) override {
    for (const PageCopy &c : copies) {
      content.at(c.to) = content.at(c.from);
      log.push_back(c);
    }
  }
  uint64_t budgetPages = ~0ull;
  std::vector<uint64_t> content;
  std::vector<PageCopy> log;

private:
  uint32_t pages_;
  uint64_t bytes_;
  uint32_t extent_;
  std::vector<bool> allocated_;
};

} // namespace rkb::kv
