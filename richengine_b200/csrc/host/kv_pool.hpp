// kv_pool.hpp — the page allocator: sole owner of page references and of which
// extents hold memory.
//
// Behaviour follows the reference allocator (runtime/engine/cache/KvPool.hpp:64-185,
// KvPool.cpp:35-413) closely enough that a random operation trace yields the same
// page ids, refusals, moves and snapshots (tests/test_host_pool.py runs both side by
// side): requests hold counted references, the prefix cache owns a page once, free
// pages come from the allocated extent with the most live pages (ties: lowest index),
// a fresh extent hands out its lowest page first, a released page is reused before
// older free pages of its extent, only empty extents are released, and compactExtent
// empties the least-used extent into the free pages of the others.
#pragma once

#include "kv_layout.hpp"

#include <cstdint>
#include <limits>
#include <span>
#include <vector>

namespace rkb::engine {

struct KvPoolSnapshot {
  uint32_t pagesAllocated = 0, pagesFree = 0, pagesActive = 0, pagesPrefix = 0;
  uint64_t allocatedBytes = 0, reclaimableBytes = 0;
  uint64_t extentAllocations = 0, extentReleases = 0;
  double extentAllocateMaxMilliseconds = 0.0, extentReleaseMaxMilliseconds = 0.0;
  uint64_t extentCompactions = 0, pagesMoved = 0;
};

// Where the pages of an emptied extent went.
struct KvPageMoves final {
  uint32_t firstPage = 0;
  std::vector<uint32_t> destinations; // by offset in the extent; the page itself where it was free
  bool empty() const noexcept { return destinations.empty(); }
  uint32_t follow(uint32_t page) const noexcept {
    return page >= firstPage && page - firstPage < destinations.size() ? destinations[page - firstPage] : page;
  }
};

struct KvPageAcquisition {
  std::vector<uint32_t> pages;
  AllocationFailure failure = AllocationFailure::None;
  bool granted() const noexcept { return failure == AllocationFailure::None; }
};

class KvPool final {
public:
  // Allocates the extents that hold pages [0, runwayPages); throws std::runtime_error when the
  // storage refuses one, std::invalid_argument for an invalid storage or runway.
  KvPool(kv::ExtentStorage &storage, uint32_t runwayPages);

  KvPageAcquisition acquirePages(uint32_t count); // each page comes with one active reference
  void retainPage(uint32_t page, bool prefixOwner);
  void releasePage(uint32_t page, bool prefixOwner);

  uint32_t pageCount() const noexcept { return uint32_t(pages_.size()); }
  uint64_t bytesPerPage() const noexcept { return storage_.bytesPerPage(); }
  uint32_t extentPages() const noexcept { return extentPages_; }
  uint32_t freePageCount() const noexcept { return freePages_; }
  bool pageActive(uint32_t page) const { return pages_.at(page).active != 0; }
  uint32_t activeReferences(uint32_t page) const { return pages_.at(page).active; }
  bool prefixOwned(uint32_t page) const { return pages_.at(page).prefix; }
  uint64_t allocatedBytes() const noexcept { return uint64_t(allocatedExtents_) * extentPages_ * bytesPerPage(); }
  uint32_t reusablePages() const noexcept { return allocatedExtents_ * extentPages_ - activePages_; }

  uint64_t reclaimEmptyExtents(bool keepRunway, uint32_t limit);
  KvPageMoves compactExtent(std::span<const uint32_t> fixed);
  KvPoolSnapshot snapshot() const;

private:
  struct Page {
    uint32_t active = 0;
    bool prefix = false;
    bool listed = false; // on its extent's free list
  };
  struct Extent {
    bool allocated = false;
    uint32_t used = 0;
    std::vector<uint32_t> freeList; // back() is handed out next
  };
  bool isFree(uint32_t page) const { return !pages_[page].active && !pages_[page].prefix; }
  uint32_t extentOf(uint32_t page) const noexcept { return page / extentPages_; }
  void listFree(uint32_t page);
  void unlistFree(uint32_t page);
  void occupy(uint32_t page);  // free -> held
  void vacate(uint32_t page);  // held -> free
  uint32_t fullestExtentWithRoom() const;
  AllocationResult growBy(uint32_t extent);
  void shrinkBy(uint32_t extent);
  void setReclaimable(uint32_t extent, bool reclaimable);

  kv::ExtentStorage &storage_;
  uint32_t extentPages_ = 0;
  std::vector<Page> pages_;
  std::vector<Extent> extents_;
  std::vector<uint32_t> reclaimable_; // empty allocated extents, most recently emptied last
  uint32_t freePages_ = 0, activePages_ = 0, prefixPages_ = 0, allocatedExtents_ = 0;
  KvPoolSnapshot counters_;
};

} // namespace rkb::engine
