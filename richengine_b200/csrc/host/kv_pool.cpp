#include "kv_pool.hpp"

#include <algorithm>
#include <chrono>
#include <stdexcept>
#include <string>

namespace rkb::engine {

namespace {
double millisecondsSince(std::chrono::steady_clock::time_point start) {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - start).count();
}
} // namespace

KvPool::KvPool(kv::ExtentStorage &storage, uint32_t runwayPages)
    : storage_(storage), extentPages_(storage.extentPages()), pages_(storage.pageCount()) {
  if (pages_.empty() || !storage_.bytesPerPage() || !extentPages_ || pages_.size() % extentPages_)
    throw std::invalid_argument("invalid KV extent storage");
  if (runwayPages > pages_.size()) throw std::invalid_argument("the KV runway exceeds the page pool");
  extents_.resize(pages_.size() / extentPages_);
  for (uint32_t extent = 0; uint64_t(extent) * extentPages_ < runwayPages; ++extent)
    if (!growBy(extent)) throw std::runtime_error("unable to allocate the KV runway");
}

// ---- free lists -------------------------------------------------------------------------------
void KvPool::listFree(uint32_t page) {
  extents_[extentOf(page)].freeList.push_back(page);
  pages_[page].listed = true;
  ++freePages_;
}

void KvPool::unlistFree(uint32_t page) {
  auto &list = extents_[extentOf(page)].freeList;
  // The common case is the page handed out next; an arbitrary page leaves when a free page is retained.
  auto at = list.back() == page ? list.end() - 1 : std::find(list.begin(), list.end(), page);
  list.erase(at);
  pages_[page].listed = false;
  --freePages_;
}

void KvPool::occupy(uint32_t page) {
  if (pages_[page].listed) unlistFree(page);
  Extent &extent = extents_[extentOf(page)];
  if (!extent.used) setReclaimable(extentOf(page), false);
  ++extent.used;
}

void KvPool::vacate(uint32_t page) {
  Extent &extent = extents_[extentOf(page)];
  --extent.used;
  listFree(page);
  if (!extent.used) setReclaimable(extentOf(page), true);
}

void KvPool::setReclaimable(uint32_t extent, bool reclaimable) {
  auto at = std::find(reclaimable_.begin(), reclaimable_.end(), extent);
  if (reclaimable && at == reclaimable_.end()) reclaimable_.push_back(extent);
  if (!reclaimable && at != reclaimable_.end()) reclaimable_.erase(at);
}

// The allocated extent with the most held pages that still has a free page; ties go to the lowest
// index, so partly used extents fill up and cold extents drain to empty.
uint32_t KvPool::fullestExtentWithRoom() const {
  uint32_t best = std::numeric_limits<uint32_t>::max();
  for (uint32_t i = 0; i < extents_.size(); ++i)
    if (!extents_[i].freeList.empty() && (best == std::numeric_limits<uint32_t>::max() || extents_[i].used > extents_[best].used))
      best = i;
  return best;
}

// ---- extents ------------------------------------------------------------------------------------
AllocationResult KvPool::growBy(uint32_t index) {
  const auto start = std::chrono::steady_clock::now();
  const AllocationResult granted = storage_.allocateExtent(index);
  if (!granted) return granted;
  ++counters_.extentAllocations;
  counters_.extentAllocateMaxMilliseconds = std::max(counters_.extentAllocateMaxMilliseconds, millisecondsSince(start));
  Extent &extent = extents_[index];
  extent.allocated = true;
  ++allocatedExtents_;
  const uint32_t first = index * extentPages_;
  for (uint32_t page = first + extentPages_; page > first;) listFree(--page); // lowest page is handed out first
  setReclaimable(index, true);
  return granted;
}

void KvPool::shrinkBy(uint32_t index) {
  const auto start = std::chrono::steady_clock::now();
  storage_.releaseExtent(index);
  ++counters_.extentReleases;
  counters_.extentReleaseMaxMilliseconds = std::max(counters_.extentReleaseMaxMilliseconds, millisecondsSince(start));
  Extent &extent = extents_[index];
  setReclaimable(index, false);
  for (uint32_t page : extent.freeList) pages_[page].listed = false;
  freePages_ -= uint32_t(extent.freeList.size());
  extent.freeList.clear();
  extent.allocated = false;
  --allocatedExtents_;
}

// ---- pages ---------------------------------------------------------------------------------------
KvPageAcquisition KvPool::acquirePages(uint32_t count) {
  if (!count) return {};
  std::vector<uint32_t> taken;
  taken.reserve(count);
  uint32_t packing = std::numeric_limits<uint32_t>::max();
  while (taken.size() < count) {
    if (freePages_) {
      // The extent being filled stays the choice until it runs out of free pages.
      if (packing == std::numeric_limits<uint32_t>::max() || extents_[packing].freeList.empty())
        packing = fullestExtentWithRoom();
      const uint32_t page = extents_[packing].freeList.back();
      unlistFree(page);
      taken.push_back(page);
      continue;
    }
    uint32_t grow = 0;
    while (grow < extents_.size() && extents_[grow].allocated) ++grow; // the lowest unallocated extent
    if (grow == extents_.size()) { // the budget must refuse growth before the page ids run out
      for (auto page = taken.rbegin(); page != taken.rend(); ++page) listFree(*page);
      throw std::logic_error("KV page ids ran out before the memory budget did");
    }
    const AllocationResult granted = growBy(grow);
    if (!granted) {
      // Everything popped goes back in reverse; extents allocated on the way stay, reclaimable.
      for (auto page = taken.rbegin(); page != taken.rend(); ++page) listFree(*page);
      return {{}, granted.failure};
    }
    packing = std::numeric_limits<uint32_t>::max();
  }
  for (uint32_t page : taken) {
    occupy(page);
    pages_[page].active = 1;
    ++activePages_;
  }
  return {std::move(taken), AllocationFailure::None};
}

void KvPool::retainPage(uint32_t page, bool prefixOwner) {
  Page &record = pages_.at(page);
  if (!extents_[extentOf(page)].allocated) throw std::logic_error("cannot retain a KV page of an unallocated extent");
  if (prefixOwner && record.prefix) throw std::logic_error("KV page already belongs to a cached block");
  if (!prefixOwner && record.active == std::numeric_limits<uint32_t>::max()) throw std::overflow_error("KV page reference overflow");
  if (isFree(page)) occupy(page);
  if (prefixOwner) {
    record.prefix = true;
    ++prefixPages_;
  } else if (!record.active++) {
    ++activePages_;
  }
}

void KvPool::releasePage(uint32_t page, bool prefixOwner) {
  Page &record = pages_.at(page);
  if (prefixOwner ? !record.prefix : !record.active) throw std::logic_error("invalid KV page release");
  if (prefixOwner) {
    record.prefix = false;
    --prefixPages_;
  } else if (!--record.active) {
    --activePages_;
  }
  if (isFree(page)) vacate(page);
}

uint64_t KvPool::reclaimEmptyExtents(bool keepRunway, uint32_t limit) {
  uint32_t released = 0;
  bool kept = false;
  // Most recently emptied first; the first one visited is the runway that stays warm.
  std::vector<uint32_t> order(reclaimable_.rbegin(), reclaimable_.rend());
  for (uint32_t extent : order) {
    if (released >= limit) break;
    if (keepRunway && !kept) { kept = true; continue; }
    shrinkBy(extent);
    ++released;
  }
  return uint64_t(released) * extentPages_ * bytesPerPage();
}

KvPageMoves KvPool::compactExtent(std::span<const uint32_t> fixed) {
  constexpr uint32_t none = std::numeric_limits<uint32_t>::max();
  uint32_t roomInUse = 0; // free pages of extents that hold pages: an empty extent is never filled
  for (const Extent &extent : extents_)
    if (extent.allocated && extent.used) roomInUse += uint32_t(extent.freeList.size());
  uint32_t emptied = none;
  for (uint32_t i = 0; i < extents_.size(); ++i) {
    const Extent &extent = extents_[i];
    if (!extent.allocated || !extent.used || extent.used > roomInUse - extent.freeList.size()) continue;
    if (emptied != none && extent.used >= extents_[emptied].used) continue;
    if (std::none_of(fixed.begin(), fixed.end(), [&](uint32_t page) { return extentOf(page) == i; })) emptied = i;
  }
  if (emptied == none) return {};

  std::vector<uint32_t> receivers;
  for (uint32_t i = 0; i < extents_.size(); ++i)
    if (i != emptied && extents_[i].allocated && extents_[i].used && !extents_[i].freeList.empty()) receivers.push_back(i);
  std::stable_sort(receivers.begin(), receivers.end(), [&](uint32_t a, uint32_t b) { return extents_[a].used > extents_[b].used; });

  // Destinations in hand-out order of each receiver, fullest receiver first.
  std::vector<uint32_t> room;
  for (uint32_t r : receivers) room.insert(room.end(), extents_[r].freeList.rbegin(), extents_[r].freeList.rend());
  const uint32_t first = emptied * extentPages_;
  std::vector<kv::PageCopy> copies;
  size_t next = 0;
  for (uint32_t page = first; page < first + extentPages_; ++page)
    if (!isFree(page)) copies.push_back({page, room[next++]});

  storage_.copyPages(copies);
  KvPageMoves moves{first, std::vector<uint32_t>(extentPages_)};
  for (uint32_t i = 0; i < extentPages_; ++i) moves.destinations[i] = first + i;
  for (const kv::PageCopy &copy : copies) {
    occupy(copy.to);
    pages_[copy.to].active = pages_[copy.from].active;
    pages_[copy.to].prefix = pages_[copy.from].prefix;
    pages_[copy.from].active = 0;
    pages_[copy.from].prefix = false;
    vacate(copy.from);
    moves.destinations[copy.from - first] = copy.to;
  }
  ++counters_.extentCompactions;
  counters_.pagesMoved += copies.size();
  return moves;
}

KvPoolSnapshot KvPool::snapshot() const {
  KvPoolSnapshot result = counters_;
  result.pagesAllocated = allocatedExtents_ * extentPages_;
  result.pagesFree = freePages_;
  result.pagesActive = activePages_;
  result.pagesPrefix = prefixPages_;
  result.allocatedBytes = allocatedBytes();
  result.reclaimableBytes = uint64_t(reclaimable_.size()) * extentPages_ * bytesPerPage();
  return result;
}

} // namespace rkb::engine
