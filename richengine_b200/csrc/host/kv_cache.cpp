#include "kv_cache.hpp"

#include <algorithm>
#include <cstring>
#include <map>
#include <stdexcept>
#include <utility>

namespace rkb::engine {

namespace {
uint64_t mix(uint64_t hash, uint64_t value) noexcept {
  return hash ^ (value + 0x9e3779b97f4a7c15ull + (hash << 6) + (hash >> 2));
}
// Sorted, disjoint spans: those that end at or before a block end before every later block too (spansFrom, Cache.cpp:19-22).
std::span<const ImageSpan> spansFrom(std::span<const ImageSpan> images, uint64_t blockBegin) {
  const auto ended = [&](const ImageSpan &span) { return span.end() <= blockBegin; };
  return {std::partition_point(images.begin(), images.end(), ended), images.end()};
}

uint64_t blockHash(uint64_t parentHash, std::span<const uint32_t> tokens, ImageIdentity images) noexcept {
  uint64_t hash = mix(0x6a09e667f3bcc909ull, parentHash);
  for (uint32_t token : tokens) hash = mix(hash, token);
  return mix(mix(hash, images.lo), images.hi);
}
} // namespace

ImageIdentity blockImageIdentity(uint64_t blockBegin, uint32_t blockTokens, std::span<const ImageSpan> spans) noexcept {
  ImageIdentity identity;
  const uint64_t blockEnd = blockBegin + blockTokens;
  for (const ImageSpan &span : spans) {
    if (span.offset >= blockEnd) break;
    if (span.end() <= blockBegin) continue;
    uint64_t lo = identity.lo ? identity.lo : 0x243f6a8885a308d3ull;
    uint64_t hi = identity.hi ? identity.hi : 0x13198a2e03707344ull;
    for (uint64_t value : {span.digestLo, span.digestHi, (uint64_t(span.gridHeight) << 32) | span.gridWidth,
                           (uint64_t(span.offset) << 32) | span.tokens, blockBegin}) {
      lo = mix(lo, value);
      hi = mix(hi, ~value);
    }
    identity = {lo, hi};
  }
  return identity;
}

// ============================== PrefixIndex ====================================================
PrefixIndex::~PrefixIndex() {
  for (auto &[id, block] : blocks_)
    if (block.page != noPage) pool_.releasePage(block.page, true);
}

PrefixIndex::Block &PrefixIndex::at(uint64_t block) {
  auto found = blocks_.find(block);
  if (found == blocks_.end()) throw std::out_of_range("unknown KV cache block");
  return found->second;
}
const PrefixIndex::Block &PrefixIndex::at(uint64_t block) const {
  auto found = blocks_.find(block);
  if (found == blocks_.end()) throw std::out_of_range("unknown KV cache block");
  return found->second;
}

void PrefixIndex::refresh(uint64_t block) {
  auto found = blocks_.find(block);
  if (found == blocks_.end()) return;
  Block &entry = found->second;
  // a poisoned block is in no order: it leaves through erasePoisonedLeaf, not as a victim (KvCache::reindex)
  const bool eligible = entry.page != noPage && !entry.residentChildren && !entry.activeUsers && !entry.transferring && !entry.poisoned;
  if (entry.listed && (!eligible || entry.listedAt != entry.lastUsed)) {
    idleLeaves_.erase({entry.listedAt, block});
    entry.listed = false;
  }
  if (eligible && !entry.listed) {
    idleLeaves_.emplace(entry.lastUsed, block);
    entry.listed = true;
    entry.listedAt = entry.lastUsed;
  }
  // the orders a full tier makes room in (KvCache::reindex, KvCache.cpp:577-592)
  uint8_t wanted = 0;
  if (entry.slot && !entry.activeUsers && !entry.transferring && !entry.poisoned)
    wanted = entry.page != noPage ? 1 : (!entry.children ? 2 : 0);
  if (entry.tierListed && (entry.tierListed != wanted || entry.tierListedAt != entry.lastUsed)) {
    (entry.tierListed == 1 ? duplicates_ : tierLeaves_).erase({entry.tierListedAt, block});
    entry.tierListed = 0;
  }
  if (wanted && !entry.tierListed) {
    (wanted == 1 ? duplicates_ : tierLeaves_).emplace(entry.lastUsed, block);
    entry.tierListed = wanted;
    entry.tierListedAt = entry.lastUsed;
  }
}

void PrefixIndex::setSlot(uint64_t block, std::shared_ptr<KvTierSlot> slot) {
  Block &entry = at(block);
  if (!slot && entry.page == noPage) throw std::logic_error("a tier-only KV cache block is erased, not stripped");
  entry.slot = std::move(slot);
  refresh(block);
}

std::optional<PrefixIndex::Candidate> PrefixIndex::tierCandidate(bool duplicate, const Candidate *after) const {
  const auto &order = duplicate ? duplicates_ : tierLeaves_;
  auto next = after ? order.upper_bound({after->lastUsed, after->block}) : order.begin();
  if (next == order.end()) return std::nullopt;
  return Candidate{next->second, next->first};
}

std::vector<uint64_t> PrefixIndex::subtree(uint64_t block) const {
  // Blocks keep no list of their children: one pass gathers them. This runs only when a tier has closed or a
  // restore has failed.
  std::unordered_map<uint64_t, std::vector<uint64_t>> below;
  for (const auto &[id, entry] : blocks_)
    if (entry.parent) below[entry.parent].push_back(id);
  // Siblings newest first, as the reference links them (a new child becomes its parent's first): with the stack below
  // the oldest child's subtree is listed first, which fixes the order pages return to the pool in.
  for (auto &[parent, children] : below) std::sort(children.begin(), children.end(), std::greater<uint64_t>());
  std::vector<uint64_t> order;
  std::vector<std::pair<uint64_t, bool>> pending{{block, false}};
  while (!pending.empty()) {
    const auto [id, expanded] = pending.back();
    pending.pop_back();
    if (expanded) {
      if (id != block) order.push_back(id);
      continue;
    }
    const Block &entry = at(id);
    if (id != block && (entry.transferring || entry.activeUsers)) return {};
    pending.push_back({id, true});
    if (auto children = below.find(id); children != below.end())
      for (uint64_t child : children->second) pending.push_back({child, false});
  }
  return order;
}

std::optional<PrefixIndex::Match> PrefixIndex::find(uint64_t parent, std::span<const uint32_t> tokens, ImageIdentity images) const {
  if (tokens.size() != pageTokens) return std::nullopt;
  if (parent && !blocks_.count(parent)) return std::nullopt;
  const uint64_t hash = blockHash(parent ? at(parent).hash : 0, tokens, images);
  const auto [first, last] = index_.equal_range(hash);
  for (auto candidate = first; candidate != last; ++candidate) {
    const Block &entry = at(candidate->second);
    // The hash only filters; a hit needs the complete key.
    if (!entry.poisoned && entry.parent == parent && entry.images == images &&
        std::equal(entry.tokens.begin(), entry.tokens.end(), tokens.begin()))
      return Match{entry.id, entry.page};
  }
  return std::nullopt;
}

PrefixIndex::Match PrefixIndex::insert(uint64_t parent, std::span<const uint32_t> tokens, uint32_t page, ImageIdentity images) {
  if (tokens.size() != pageTokens) throw std::invalid_argument("KV cache block must contain one full page");
  if (page >= pool_.pageCount()) throw std::out_of_range("KV cache physical page is out of range");
  if (auto existing = find(parent, tokens, images)) {
    Match result = *existing;
    if (existing->page == noPage) {
      adoptPage(existing->id, page);
      result.page = page;
    } else if (at(existing->id).transferring) {
      result.page = page; // its page is still being filled; the writer keeps its own copy
    }
    return result;
  }
  if (parent && !blocks_.count(parent)) throw std::invalid_argument("KV cache parent block is unknown");
  if (parent && at(parent).page == noPage) throw std::logic_error("KV cache parent block has no page");
  if (blockOnPage_[page]) throw std::logic_error("KV cache page already holds a block");
  Block entry;
  entry.id = nextId_++;
  entry.parent = parent;
  entry.hash = blockHash(parent ? at(parent).hash : 0, tokens, images);
  std::copy(tokens.begin(), tokens.end(), entry.tokens.begin());
  entry.images = images;
  entry.page = page;
  entry.lastUsed = ++clock_;
  pool_.retainPage(page, true);
  const uint64_t id = entry.id;
  index_.emplace(entry.hash, id);
  blocks_.emplace(id, std::move(entry));
  blockOnPage_[page] = id;
  ++resident_;
  if (parent) {
    Block &above = at(parent);
    ++above.children;
    ++above.residentChildren;
    refresh(parent);
  }
  refresh(id);
  ++generation_;
  return {id, page};
}

// Recency as the reference keeps it (KvCache::retainActive / releaseActive, KvCache.cpp:227-249): a block is stamped
// when a user takes it; a released leaf is the newest, a parent keeps the recency its children pass on.
void PrefixIndex::retainActive(uint64_t block) {
  Block &entry = at(block);
  ++entry.activeUsers;
  entry.lastUsed = ++clock_;
  refresh(block);
}
void PrefixIndex::releaseActive(uint64_t block) noexcept {
  auto found = blocks_.find(block);
  if (found == blocks_.end()) return;
  Block &entry = found->second;
  if (entry.activeUsers) --entry.activeUsers;
  if (!entry.activeUsers && !entry.children) entry.lastUsed = ++clock_;
  refresh(block);
  erasePoisonedLeaf(block);
}
// A parent that has just become a leaf no request holds is as warm as the child it lost (KvCache::inherit,
// KvCache.cpp:441-446).
void PrefixIndex::inherit(Block &parent, uint64_t lastUsed) noexcept {
  const bool leaf = parent.page != noPage ? !parent.residentChildren : !parent.children;
  if (leaf && !parent.activeUsers) parent.lastUsed = std::max(parent.lastUsed, lastUsed);
}
void PrefixIndex::touch(uint64_t block) noexcept {
  auto found = blocks_.find(block);
  if (found != blocks_.end()) found->second.lastUsed = ++clock_;
  refresh(block);
}

PrefixIndex::Chain PrefixIndex::chain(uint64_t block) const {
  Chain result;
  for (uint64_t id = block; id; id = at(id).parent) {
    result.blocks.push_back(id);
    result.pages.push_back(at(id).page);
  }
  std::reverse(result.blocks.begin(), result.blocks.end());
  std::reverse(result.pages.begin(), result.pages.end());
  return result;
}

void PrefixIndex::dropPage(uint64_t block) {
  Block &entry = at(block);
  if (entry.page == noPage || entry.residentChildren || entry.activeUsers || !entry.slot)
    throw std::logic_error("only an idle resident leaf with a tier copy can drop its page");
  blockOnPage_[entry.page] = 0;
  pool_.releasePage(entry.page, true);
  entry.page = noPage;
  --resident_;
  if (entry.parent) {
    Block &above = at(entry.parent);
    --above.residentChildren;
    inherit(above, entry.lastUsed);
    refresh(entry.parent);
  }
  refresh(block);
}

bool PrefixIndex::abandonRestore(uint64_t block) {
  Block &entry = at(block);
  if (!entry.transferring || entry.residentChildren || entry.activeUsers) return false;
  entry.transferring = false;
  dropPage(block);
  return true;
}

void PrefixIndex::adoptPage(uint64_t block, uint32_t page) {
  Block &entry = at(block);
  if (entry.page != noPage) throw std::logic_error("KV cache block already has a page");
  if (entry.parent && at(entry.parent).page == noPage) throw std::logic_error("the parent block must be resident first");
  if (blockOnPage_.at(page)) throw std::logic_error("KV cache page already holds a block");
  pool_.retainPage(page, true);
  entry.page = page;
  blockOnPage_[page] = block;
  ++resident_;
  if (entry.parent) {
    ++at(entry.parent).residentChildren;
    refresh(entry.parent);
  }
  refresh(block);
}

bool PrefixIndex::adoptTierBlock(uint64_t id, uint64_t parent, std::span<const uint32_t> tokens, ImageIdentity images,
                                 std::shared_ptr<KvTierSlot> slot, uint64_t lastUsed) {
  if (!id || id == ~0ull || blocks_.count(id) || tokens.size() != pageTokens || !slot) throw std::invalid_argument("invalid adopted KV cache block");
  if (parent && !blocks_.count(parent)) throw std::invalid_argument("adopted KV cache block's parent is unknown");
  if (find(parent, tokens, images)) return false;
  Block entry;
  entry.id = id;
  entry.parent = parent;
  entry.hash = blockHash(parent ? at(parent).hash : 0, tokens, images);
  std::copy(tokens.begin(), tokens.end(), entry.tokens.begin());
  entry.images = images;
  entry.lastUsed = lastUsed;
  entry.slot = std::move(slot);
  index_.emplace(entry.hash, id);
  blocks_.emplace(id, std::move(entry));
  if (parent) { ++at(parent).children; refresh(parent); }
  refresh(id);
  nextId_ = std::max(nextId_, id + 1);
  ++generation_;
  return true;
}

void PrefixIndex::continueAfter(uint64_t highestId, uint64_t lastUsed) noexcept {
  nextId_ = std::max(nextId_, highestId + 1);
  clock_ = std::max(clock_, lastUsed);
}

std::vector<std::pair<model::KvBlockLabel, std::shared_ptr<KvTierSlot>>> PrefixIndex::tierCopies() const {
  std::vector<std::pair<model::KvBlockLabel, std::shared_ptr<KvTierSlot>>> copies;
  for (const auto &[id, block] : blocks_) {
    if (!block.slot || block.poisoned) continue;
    if (block.transferring && block.page != noPage) continue; // a demotion that has not landed yet
    model::KvBlockLabel label{block.id, block.parent, block.lastUsed, block.images.lo, block.images.hi, block.tokens};
    copies.emplace_back(label, block.slot);
  }
  std::sort(copies.begin(), copies.end(), [](const auto &a, const auto &b) { return a.first.id < b.first.id; });
  return copies;
}

void PrefixIndex::followPages(const KvPageMoves &moves) noexcept {
  for (uint32_t offset = 0; offset < moves.destinations.size(); ++offset) {
    const uint32_t from = moves.firstPage + offset, to = moves.destinations[offset];
    if (from == to || !blockOnPage_[from]) continue;
    const uint64_t id = blockOnPage_[from];
    blockOnPage_[from] = 0;
    blockOnPage_[to] = id;
    blocks_.find(id)->second.page = to;
  }
}

// It matches no lookup from now on, and the copy that failed to read is given up (KvCache::poison, KvCache.cpp:469-478).
void PrefixIndex::poison(uint64_t block) {
  Block &entry = at(block);
  entry.poisoned = true;
  ++generation_;
  entry.slot.reset();
  refresh(block);
  erasePoisonedLeaf(block);
}

void PrefixIndex::erasePoisonedLeaf(uint64_t block) noexcept {
  auto found = blocks_.find(block);
  if (found == blocks_.end() || !found->second.poisoned || found->second.children || found->second.activeUsers ||
      found->second.transferring)
    return;
  try { erase(block); } catch (...) { std::terminate(); }
}

// KvCache::erase (KvCache.cpp:515-558), in its order: the block leaves the graph, its parent inherits its recency and,
// if it is a poisoned block nothing hangs on any more, leaves too (and so on up the chain); the page returns to the pool
// last, after the pages of the ancestors that left with it.
void PrefixIndex::erase(uint64_t block) {
  Block &entry = at(block);
  if (entry.children || entry.activeUsers || entry.transferring)
    throw std::logic_error("only a block without children, users or transfer can be removed");
  const uint64_t parent = entry.parent, lastUsed = entry.lastUsed, hash = entry.hash;
  const uint32_t page = entry.page;
  if (entry.listed) idleLeaves_.erase({entry.listedAt, block});
  if (entry.tierListed) (entry.tierListed == 1 ? duplicates_ : tierLeaves_).erase({entry.tierListedAt, block});
  const auto [first, last] = index_.equal_range(hash);
  for (auto it = first; it != last; ++it)
    if (it->second == block) { index_.erase(it); break; }
  blocks_.erase(block);
  ++generation_;
  if (page != noPage) {
    blockOnPage_[page] = 0;
    --resident_;
  }
  if (parent) {
    Block &above = at(parent);
    --above.children;
    if (page != noPage) --above.residentChildren;
    inherit(above, lastUsed);
    refresh(parent);
    erasePoisonedLeaf(parent);
  }
  if (page != noPage) pool_.releasePage(page, true);
}

std::optional<PrefixIndex::Candidate> PrefixIndex::evictionCandidate() const {
  if (idleLeaves_.empty()) return std::nullopt;
  return Candidate{idleLeaves_.begin()->second, idleLeaves_.begin()->first};
}

std::optional<PrefixIndex::Candidate> PrefixIndex::evictionCandidate(const Candidate *after, const std::function<bool(uint64_t)> &accept) const {
  auto next = after ? idleLeaves_.upper_bound({after->lastUsed, after->block}) : idleLeaves_.begin();
  for (; next != idleLeaves_.end(); ++next)
    if (accept(next->second)) return Candidate{next->second, next->first};
  return std::nullopt;
}

void PrefixIndex::adjustStatesBelow(uint64_t block, int states, int inUse) {
  for (uint64_t id = at(block).parent; id; id = at(id).parent) {
    Block &above = at(id);
    above.statesBelow = uint32_t(int(above.statesBelow) + states);
    above.statesInUseBelow = uint32_t(int(above.statesInUseBelow) + inUse);
  }
}

uint32_t PrefixIndex::tierBlocks() const noexcept {
  uint32_t count = 0;
  for (const auto &[id, entry] : blocks_) count += entry.slot != nullptr;
  return count;
}

// ================================== Cache ========================================================
Cache::~Cache() {
  // Transfers read or write their pages in place: they retire before the pages can go.
  const auto drain = [this](Transfer &t) {
    if (t.ticket) { // a restore that was never submitted has no IO to drain
      while (!t.ticket->ready()) tier_->poll();
      t.ticket->finish();
    }
    if (index_.contains(t.block)) index_.setTransferring(t.block, false);
  };
  for (Transfer &t : demotions_) drain(t);
  for (auto &[block, t] : restores_) drain(t);
  for (auto &[id, active] : requests_) {
    for (uint32_t page : active.pages) pool_.releasePage(page, false);
    if (!active.blocks.empty()) index_.releaseActive(active.blocks.back());
  }
}

Cache::Request &Cache::request(uint64_t id) {
  auto found = requests_.find(id);
  if (found == requests_.end()) throw std::invalid_argument("unknown request id");
  return found->second;
}
const Cache::Request &Cache::request(uint64_t id) const {
  auto found = requests_.find(id);
  if (found == requests_.end()) throw std::invalid_argument("unknown request id");
  return found->second;
}

void Cache::beginRequest(uint64_t id) {
  if (!id) throw std::invalid_argument("invalid request id");
  if (!requests_.emplace(id, Request{}).second) throw std::invalid_argument("duplicate request id");
}

void Cache::endRequest(uint64_t id) {
  auto found = requests_.find(id);
  if (found == requests_.end()) return;
  for (uint32_t page : found->second.pages) pool_.releasePage(page, false);
  if (!found->second.blocks.empty()) index_.releaseActive(found->second.blocks.back());
  // Reads that were never submitted have no IO to drain: their pages return leaf first, unless another request
  // waits for the block, a block below it is resident, or a state was published on it meanwhile (Cache::endRequest,
  // Cache.cpp:160-175; KvCache::abandonRestore, KvCache.cpp:411-418).
  const std::vector<uint64_t> &chain = found->second.blocks;
  if (found->second.pendingRestores)
    for (uint64_t block : chain)
      if (auto waited = restores_.find(block); waited != restores_.end()) std::erase(waited->second.waiters, id);
  // only a request that waited for reads takes any back
  for (auto block = chain.rbegin(); found->second.pendingRestores && block != chain.rend() && !restores_.empty(); ++block) {
    auto queued = restores_.find(*block);
    if (queued == restores_.end() || queued->second.ticket || !queued->second.waiters.empty() || states_.stateResident(*block)) continue;
    if (!index_.contains(*block)) continue; // a poisoned tip left with the request's hold on it
    if (!index_.abandonRestore(*block)) continue;
    restores_.erase(queued);
    --counters_.restores;
    ++counters_.cancelledRestores;
  }
  requests_.erase(found);
  dropPoisoned(); // a block whose restore failed leaves once its last request has let go
}

TokenAdmission Cache::admitPages(uint32_t count, std::vector<uint32_t> &pages) {
  KvPageAcquisition acquired = pool_.acquirePages(count);
  if (!acquired.granted()) {
    // Demoted pages free theirs when their copies land: wait once those on their way cover what
    // the free pages do not; until then the caller reclaims (Cache.cpp:400-413).
    const uint32_t missing = count - std::min(count, pool_.freePageCount());
    const uint32_t pending = pendingPages();
    const bool covered = pending > 0 && pending >= missing;
    return {covered ? TokenAdmissionFailure::Pending : TokenAdmissionFailure::Denied, count, pool_.freePageCount(), acquired.failure};
  }
  pages = std::move(acquired.pages);
  return {};
}

TokenAdmission Cache::ensureTokens(uint64_t id, uint64_t tokenCount) {
  Request &active = request(id);
  const uint64_t needed = (tokenCount + kv::kPageTokens - 1) / kv::kPageTokens;
  if (needed > 0xffffffffull) throw std::invalid_argument("KV target exceeds the page id range");
  const uint32_t previous = uint32_t(active.pages.size());
  if (needed <= previous) return {};
  std::vector<uint32_t> acquired;
  if (const TokenAdmission admission = admitPages(uint32_t(needed) - previous, acquired); !admission.granted()) return admission;
  active.pages.insert(active.pages.end(), acquired.begin(), acquired.end());
  changed(active, previous);
  return {};
}

PageTableView Cache::pageTable(uint64_t id) const {
  const Request &active = request(id);
  return {active.pages, active.revision, active.firstChanged};
}

void Cache::publishCommittedBlocks(uint64_t id, std::span<const uint32_t> exactTokens, uint32_t committedTokens,
                                   std::span<const ImageSpan> images) {
  Request &active = request(id);
  if (committedTokens > exactTokens.size()) throw std::invalid_argument("committed KV exceeds exact token history");
  const uint32_t fullBlocks = committedTokens / kv::kPageTokens;
  if ((uint64_t(committedTokens) + kv::kPageTokens - 1) / kv::kPageTokens > active.pages.size())
    throw std::logic_error("committed KV has no physical request page");
  if (fullBlocks < active.blocks.size()) throw std::logic_error("committed KV history moved backwards");
  while (active.blocks.size() < fullBlocks) {
    const uint32_t logical = uint32_t(active.blocks.size());
    const uint64_t parent = logical ? active.blocks.back() : 0;
    const uint32_t writerPage = active.pages[logical];
    const uint32_t begin = logical * kv::kPageTokens;
    images = spansFrom(images, begin);
    const PrefixIndex::Match placed = index_.insert(parent, exactTokens.subspan(begin, kv::kPageTokens), writerPage,
                                                    blockImageIdentity(begin, kv::kPageTokens, images));
    const bool replace = placed.page != writerPage;
    if (replace) pool_.retainPage(placed.page, false);
    index_.retainActive(placed.id);
    active.blocks.push_back(placed.id);
    if (replace) { // identical content already lives on another page: move onto it
      active.pages[logical] = placed.page;
      changed(active, logical);
      pool_.releasePage(writerPage, false);
    }
    if (parent) index_.releaseActive(parent);
  }
}

// Extends a chain that matches the prompt's first pages by the pages that follow, at most (n-1)/32 in all; returns
// the pages hashed (Cache::extendMatch, Cache.cpp:179-199).
size_t Cache::extendMatch(std::vector<uint64_t> &blocks, std::span<const uint32_t> prompt, std::span<const ImageSpan> images) const {
  if (prompt.empty()) return 0;
  const size_t maximum = (prompt.size() - 1) / kv::kPageTokens; // one real token stays to recompute
  size_t hashed = 0;
  for (size_t i = blocks.size(); i < maximum; ++i) {
    ++hashed;
    images = spansFrom(images, i * kv::kPageTokens);
    auto match = index_.find(blocks.empty() ? 0 : blocks.back(), prompt.subspan(i * kv::kPageTokens, kv::kPageTokens),
                             blockImageIdentity(i * kv::kPageTokens, kv::kPageTokens, images));
    if (!match) break;
    blocks.push_back(match->id);
  }
  return hashed;
}

// Tokens up to the deepest state on a chain (Cache::stateTokens, Cache.cpp:201-207).
uint32_t Cache::stateTokens(std::span<const uint64_t> blocks) const {
  for (size_t i = blocks.size(); i > 0; --i)
    if (states_.contains(blocks[i - 1])) return uint32_t(i * kv::kPageTokens);
  return 0;
}

Cache::Probe Cache::probe(std::span<const uint32_t> prompt, std::span<const ImageSpan> images) {
  Probe result;
  result.owner_ = this;
  result.generation_ = index_.generation();
  lookups_.probeHashedBlocks += extendMatch(result.blocks_, prompt, images);
  result.cachedTokens_ = stateTokens(result.blocks_);
  return result;
}

void Cache::refresh(Probe &probe, std::span<const uint32_t> prompt, std::span<const ImageSpan> images) {
  if (probe.owner_ != this) throw std::logic_error("a scheduling probe belongs to another cache");
  if (probe.generation_ != index_.generation()) {
    auto cut = std::find_if(probe.blocks_.begin(), probe.blocks_.end(), [&](uint64_t block) { return !index_.matchable(block); });
    probe.blocks_.erase(cut, probe.blocks_.end());
    lookups_.probeHashedBlocks += extendMatch(probe.blocks_, prompt, images);
    probe.generation_ = index_.generation();
  }
  probe.cachedTokens_ = stateTokens(probe.blocks_); // states come and go without a change of the graph
}

std::vector<uint64_t> Cache::lookup(std::span<const uint32_t> prompt, const Probe *probe, std::span<const ImageSpan> images) {
  std::vector<uint64_t> blocks;
  if (probe && probe->owner_ == this && probe->generation_ == index_.generation()) blocks = probe->blocks_;
  else extendMatch(blocks, prompt, images);
  if (!blocks.empty()) {
    index_.touch(blocks.back());
    // A chain that ends in tier-only blocks keeps its resident boundary as warm as its tip: a restore adopts the
    // blocks below it (Cache.cpp:248-257).
    auto resident = std::find_if(blocks.rbegin(), blocks.rend(), [&](uint64_t block) { return index_.page(block) != PrefixIndex::noPage; });
    if (resident != blocks.rbegin() && resident != blocks.rend()) index_.touch(*resident);
  }
  return blocks;
}

Cache::StateLookup Cache::lookupWithState(std::span<const uint32_t> prompt, const Probe *probe, std::span<const ImageSpan> images) {
  StateLookup result;
  result.blocks = lookup(prompt, probe, images);
  const std::vector<uint64_t> &blocks = result.blocks;
  if (blocks.empty()) return result;
  result.kvBoundary = uint32_t(blocks.size() * kv::kPageTokens);
  for (size_t i = blocks.size(); i-- > 0;) // the deepest state on the chain (StateCache::acquireDeepest)
    if (states_.contains(blocks[i])) {
      result.stateBlock = blocks[i];
      result.resumeBoundary = uint32_t((i + 1) * kv::kPageTokens);
      states_.pin(blocks[i]);
      break;
    }
  if (result.kvBoundary > result.resumeBoundary && index_.stateBelow(blocks.back())) result.junctionBoundary = result.kvBoundary;
  for (size_t i = blocks.size(); i-- > 0;) {
    if (blocks[i] == result.stateBlock) break;
    if (index_.hadState(blocks[i]) && !states_.contains(blocks[i])) {
      result.lostState = true;
      break;
    }
  }
  return result;
}

void Cache::recordLookup(const StateLookup &lookup) noexcept {
  lookups_.kvHitTokens += lookup.kvBoundary;
  if (lookup.junctionBoundary) ++lookups_.lazyJunctions;
  if (lookup.lostState) ++lookups_.lostStateMisses;
}

TokenAdmission Cache::attachPrefix(uint64_t id, std::span<const uint64_t> blocks, uint32_t *resumeTokens) {
  Request &active = request(id);
  if (!active.pages.empty() || !active.blocks.empty()) throw std::logic_error("a prefix attaches to a request without pages");
  if (resumeTokens) *resumeTokens = 0;
  if (blocks.empty()) return {};
  // Host-only blocks need fresh pages; take them all first so a refusal changes nothing.
  uint32_t missing = 0;
  for (uint64_t block : blocks) missing += index_.page(block) == PrefixIndex::noPage && !index_.transferring(block);
  std::vector<uint32_t> fresh;
  if (missing) {
    if (!tier_) throw std::logic_error("host-only blocks need a tier");
    if (const TokenAdmission admission = admitPages(missing, fresh); !admission.granted()) return admission;
  }
  size_t next = 0;
  bool refused = false; // restores start in block order and stop at the first the tier refuses
  for (uint64_t block : blocks) { // root first: a parent is resident before its child adopts a page
    uint32_t page = index_.page(block);
    if (page == PrefixIndex::noPage) {
      page = fresh[next++];
      index_.adoptPage(block, page);
      index_.setTransferring(block, true);
      Transfer restore{block, page, nullptr, index_.slot(block)};
      if (!refused && tier_->canRestore()) restore.ticket = tier_->restore(restore.slot, page);
      if (!restore.ticket) refused = true;
      restores_.emplace(block, std::move(restore)); // a refused start is retried by pollTransfers, in block order
      ++counters_.restores;
      // the pool's acquisition gave the request an active reference already
    } else {
      pool_.retainPage(page, false);
    }
    active.pages.push_back(page);
    auto pending = restores_.find(block);
    if (pending != restores_.end()) { // its own read, or one another request started: both wait for it
      pending->second.waiters.push_back(id);
      ++active.pendingRestores;
    }
  }
  active.blocks.assign(blocks.begin(), blocks.end());
  index_.retainActive(blocks.back());
  index_.touch(blocks.back());
  changed(active, 0);
  if (resumeTokens) *resumeTokens = uint32_t(blocks.size()) * kv::kPageTokens;
  return {};
}

// Cache::kvRestoreStatus (Cache.cpp:787-792): 0 = nothing to wait for, 1 = pending, 2 = a read failed (the request
// recomputes: the block matches nothing any more).
int Cache::restoreStatus(uint64_t id) const {
  const Request &active = request(id);
  if (active.restoreFailed) return 2;
  return active.pendingRestores ? 1 : 0;
}

bool Cache::restoresPending(uint64_t id) const { return request(id).pendingRestores != 0; }

uint32_t Cache::forkRequest(uint64_t parentId, uint64_t childId, uint32_t committedTokens) {
  const Request &parent = request(parentId);
  Request &child = request(childId);
  if (!child.pages.empty()) throw std::logic_error("a fork target starts without pages");
  const uint32_t fullPages = committedTokens / kv::kPageTokens;
  const bool partial = committedTokens % kv::kPageTokens != 0;
  if (fullPages + (partial ? 1u : 0u) > parent.pages.size()) throw std::logic_error("fork point lies past the parent's pages");
  std::vector<uint32_t> own;
  if (partial) {
    const TokenAdmission admission = admitPages(1, own);
    if (!admission.granted()) throw std::runtime_error("no page for the forked tail");
  }
  for (uint32_t i = 0; i < fullPages; ++i) { // full pages are immutable while shared
    pool_.retainPage(parent.pages[i], false);
    child.pages.push_back(parent.pages[i]);
  }
  const size_t cached = std::min<size_t>(parent.blocks.size(), fullPages);
  child.blocks.assign(parent.blocks.begin(), parent.blocks.begin() + cached);
  if (cached) index_.retainActive(child.blocks.back());
  uint32_t copied = 0;
  if (partial) { // both would append into this page: the child gets its own copy
    const kv::PageCopy copy{parent.pages[fullPages], own[0]};
    storage_.copyPages({&copy, 1});
    child.pages.push_back(own[0]);
    copied = 1;
    ++counters_.forkCopies;
  }
  changed(child, 0);
  return copied;
}

uint32_t Cache::truncate(uint64_t id, uint32_t committedTokens, uint32_t scratchTokens) {
  Request &active = request(id);
  const uint32_t keep = uint32_t((uint64_t(committedTokens) + scratchTokens + kv::kPageTokens - 1) / kv::kPageTokens);
  if (keep >= active.pages.size()) return 0;
  if (keep < active.blocks.size()) throw std::logic_error("published pages cannot be truncated");
  const uint32_t released = uint32_t(active.pages.size()) - keep;
  for (uint32_t i = keep; i < active.pages.size(); ++i) pool_.releasePage(active.pages[i], false);
  active.pages.resize(keep);
  changed(active, keep);
  counters_.truncatedPages += released;
  return released;
}

Cache::LeafReclaim Cache::reclaimKvLeaf(uint64_t block, bool immediate) {
  if (index_.slot(block)) { // a tier copy exists already: the page can go at once
    index_.dropPage(block);
    ++counters_.evictedBlocks;
    return LeafReclaim::Started;
  }
  // A leaf worth a copy is written (the page returns only when the copy lands); copies below that nothing needs go
  // with a leaf that is not (Cache::reclaimKvLeaf, Cache.cpp:629-659).
  if (worthACopy(block)) {
    // the tier has said "not now" in this scan already: every leaf that needs a write would hear the same
    if (immediate && tierWritable()) return LeafReclaim::Impossible;
    const LeafReclaim demotion = demoteKv(block);
    if (demotion != LeafReclaim::Impossible) return demotion;
    // A leaf its tier subtree depends on stays in RAM while the tier may still write it: dropping it would orphan
    // every copy below it. Once a failed write has closed the tier, the subtree goes with it, as without a tier.
    if ((stateCoupled_ ? index_.stateBelow(block) : index_.tierChildren(block)) && tierWritable()) return LeafReclaim::Impossible;
  }
  if (index_.tierChildren(block) && !dropTierSubtree(block)) return LeafReclaim::Impossible;
  if (index_.children(block)) return LeafReclaim::Impossible;
  states_.forget(block);
  index_.erase(block);
  ++counters_.evictedBlocks;
  return LeafReclaim::Started;
}

// Cache::demoteKv (Cache.cpp:824-851): Pending = worth waiting for (transfers in flight will make room), Impossible =
// nothing will, and the leaf goes as without a tier.
Cache::LeafReclaim Cache::demoteKv(uint64_t block) {
  if (!tierWritable()) return LeafReclaim::Impossible;
  const auto waitOrGiveUp = [this] { return transfersInFlight() ? LeafReclaim::Pending : LeafReclaim::Impossible; };
  if (!tier_->canDemote()) { // do not discard a copy for a transfer that cannot start yet
    ++counters_.demotionsRefused;
    return waitOrGiveUp();
  }
  std::shared_ptr<KvTierSlot> slot = acquireTierSlot(kvNeededByStateInUse(block));
  if (!slot) return waitOrGiveUp();
  // making room may have taken the states the leaf was kept for; it then goes like any leaf nothing needs
  if (!worthACopy(block)) return LeafReclaim::Impossible;
  std::unique_ptr<KvTransfer> ticket = tier_->demote(index_.page(block), slot);
  if (!ticket) {
    ++counters_.demotionsRefused;
    return waitOrGiveUp();
  }
  index_.setTransferring(block, true);
  demotions_.push_back({block, index_.page(block), std::move(ticket), std::move(slot)});
  ++counters_.demotions;
  return LeafReclaim::Started;
}

std::shared_ptr<KvTierSlot> Cache::acquireTierSlot(bool inUse) {
  for (;;) {
    if (auto slot = tier_->acquireSlot()) return slot;
    if (!freeTierSpace(inUse)) return {};
  }
}

// A full tier replaces by recency (Cache::freeDiskSpace, Cache.cpp:871-905, as far as KV copies go): the oldest copy
// of a page that is resident too goes first (it loses nothing), then the oldest tier-only block without children,
// with the state on it; a block that holds a state in use stays unless the writer is in use itself.
bool Cache::freeTierSpace(bool inUse) {
  if (const auto duplicate = index_.tierCandidate(true)) {
    index_.setSlot(duplicate->block, nullptr);
    ++counters_.replacedCopies;
    return true;
  }
  auto leaf = index_.tierCandidate(false);
  while (leaf && !inUse && kvNeededByStateInUse(leaf->block)) leaf = index_.tierCandidate(false, &*leaf);
  if (!leaf) return false;
  states_.forget(leaf->block);
  index_.erase(leaf->block);
  ++counters_.replacedCopies;
  ++counters_.evictedBlocks;
  return true;
}

// Everything below a block leaves with it, unless some of it is in use or in transfer (Cache::dropDiskSubtree,
// Cache.cpp:661-672).
bool Cache::dropTierSubtree(uint64_t block) {
  const std::vector<uint64_t> below = index_.subtree(block);
  if (below.empty()) return false;
  for (uint64_t id : below) {
    states_.forget(id);
    index_.erase(id);
    ++counters_.evictedBlocks;
  }
  return true;
}

// A block whose restore failed matches nothing any more; it and what hangs below it leave as soon as no request
// holds them (Cache::dropPoisoned, Cache.cpp:674-686).
void Cache::dropPoisoned() {
  std::erase_if(poisoned_, [&](uint64_t block) {
    if (!index_.contains(block)) return true;
    for (uint64_t below : index_.subtree(block)) {
      states_.forget(below);
      if (!index_.contains(below)) continue; // a poisoned block below may have left with its last child
      index_.erase(below);
      ++counters_.evictedBlocks;
    }
    return !index_.contains(block); // it leaves with its last child, user or transfer (PrefixIndex::erasePoisonedLeaf)
  });
}

// Without composite states every idle leaf is a dead leaf, and this is "the oldest idle leaf first".
bool Cache::reclaimOne() { return evictOne(ReclaimClass::InUse, false, true).madeProgress; }

uint64_t Cache::blockAt(uint64_t id, uint32_t tokens) const {
  const Request &active = request(id);
  if (!tokens || tokens % kv::kPageTokens) return 0;
  const uint32_t index = tokens / kv::kPageTokens - 1;
  return index < active.blocks.size() ? active.blocks[index] : 0;
}

void Cache::publishCompositeState(uint64_t block, uint64_t bytes, bool checkpoint) {
  if (!index_.contains(block)) throw std::invalid_argument("a composite state needs its KV block in the cache");
  if (!bytes) throw std::invalid_argument("a composite state has a size");
  states_.publish(block, bytes, checkpoint);
}

void Cache::publishStoredState(uint64_t block, uint64_t bytes, bool checkpoint) {
  if (!index_.contains(block)) throw std::invalid_argument("a composite state needs its KV block in the cache");
  if (!bytes) throw std::invalid_argument("a composite state has a size");
  states_.publishStored(block, bytes, checkpoint);
  stateWriteRetired_ = true;
}

std::optional<Cache::Victim> Cache::reclaimOldest(bool inUse, bool keepResumePoint, bool pagesOnly) {
  using Candidate = PrefixIndex::Candidate;
  // A dead leaf (no state restores through it) goes before anything a state needs; one that cannot go now stays
  // and the next goes. Once the tier has answered "not now" the scan stops asking it: the leaves that need a write
  // wait with that one, and those whose page frees at once still go (Cache::reclaimOldest, Cache.cpp:507-550).
  bool immediate = false;
  const auto step = [&](uint64_t block) {
    const LeafReclaim outcome = reclaimKvLeaf(block, immediate);
    if (outcome == LeafReclaim::Pending) immediate = true;
    return outcome == LeafReclaim::Started;
  };
  if (!inUse) {
    const auto dead = [this](uint64_t id) { return !kvNeededByState(id); };
    for (auto leaf = index_.evictionCandidate(nullptr, dead); leaf; leaf = index_.evictionCandidate(&*leaf, dead))
      if (step(leaf->block)) return Victim{true};
  }
  std::optional<StateCandidate> state;
  if (!pagesOnly) state = inUse ? states_.inUseCandidate() : states_.ordinaryCandidate(keepResumePoint);
  // the leaves a state needs (the dead ones were asked above): without a state in RAM on them (one goes first, in the
  // order every victim goes in), or with one in a page scan
  const auto needed = [&](uint64_t id) {
    return kvNeededByState(id) && (pagesOnly || !states_.stateResident(id)) && kvNeededByStateInUse(id) == inUse;
  };
  std::optional<Candidate> kv = index_.evictionCandidate(nullptr, needed);
  while (state || kv) {
    if (state && (!kv || state->lastUsed <= kv->lastUsed)) {
      if (states_.reclaim(state->block)) return Victim{false};
      state.reset();
      continue;
    }
    if (states_.stateResident(kv->block)) { // a page scan's leaf gives up its state first; the resume point stays, and its leaf
      if ((!keepResumePoint || kv->block != states_.resumePoint()) && states_.reclaim(kv->block)) return Victim{false};
      kv = index_.evictionCandidate(&*kv, needed);
      continue;
    }
    if (step(kv->block)) return Victim{true};
    kv = index_.evictionCandidate(&*kv, needed);
  }
  return std::nullopt;
}

ReclaimStep Cache::evictOne(ReclaimClass upTo, bool keepResumePoint, bool pagesOnly) {
  // Disposable checkpoints go first, except in a page scan, to which their buffers give no page.
  if (!pagesOnly)
    if (const auto oldest = states_.checkpointCandidate(keepResumePoint)) {
      uint64_t freed = 0;
      if (states_.reclaim(oldest->block, &freed)) return {true, false, true, freed};
    }
  for (const bool inUse : {false, true}) {
    if (inUse && upTo == ReclaimClass::Ordinary) break;
    if (inUse && transfersInFlight()) return {false, true, false, 0};
    const uint64_t before = states_.residentBytes();
    if (const auto victim = reclaimOldest(inUse, keepResumePoint, pagesOnly))
      return {true, false, !victim->kv, before - states_.residentBytes()};
  }
  return {false, transfersInFlight(), false, 0};
}

ReclaimStep Cache::releaseExtent(bool keepRunway) {
  if (const uint64_t bytes = pool_.reclaimEmptyExtents(keepRunway, 1)) return {true, false, false, bytes};
  if (compactExtent()) return {true, false, false, pool_.reclaimEmptyExtents(keepRunway, 1)};
  return {};
}

ReclaimStep Cache::reclaimStep(ReclaimMode mode, ReclaimClass upTo, bool keepResumePoint, bool keepRunway) {
  const bool release = mode == ReclaimMode::ReleaseExtents;
  if (release)
    if (const ReclaimStep released = releaseExtent(keepRunway); released.madeProgress) return released;
  ReclaimStep evicted = evictOne(upTo, keepResumePoint, mode == ReclaimMode::ReusePages);
  evicted.reclaimedBytes = 0; // a state's buffers return to the model's pool, not to the device: only extents count here
  if (evicted.madeProgress && release) evicted.reclaimedBytes += pool_.reclaimEmptyExtents(keepRunway, 1);
  return evicted;
}

ReclaimStep Cache::evictAll() {
  uint64_t released = releaseEmptyExtents(false);
  bool evicted = false;
  while (evictOne(ReclaimClass::InUse, false, false).madeProgress) evicted = true;
  do released += releaseEmptyExtents(false);
  while (compactExtent());
  return {evicted || released != 0, false, false, released};
}

bool Cache::reclaimOneState(bool checkpointsOnly, uint64_t forBlock) {
  const auto recycle = [this](const std::optional<StateCandidate> &state) { return state && states_.reclaim(state->block); };
  if (recycle(states_.checkpointCandidate(false))) return true;
  if (checkpointsOnly) return false;
  if (recycle(states_.ordinaryCandidate(false))) return true;
  // only a publication that is itself in use may take a state in use
  return states_.inUse(forBlock) && recycle(states_.inUseCandidate());
}

uint32_t Cache::reclaimForPages(uint32_t pages) {
  uint32_t started = 0;
  while (pool_.freePageCount() + pendingPages() < pages && reclaimOne()) ++started;
  return started;
}

void Cache::pollTransfers() {
  if (!tier_) return;
  tier_->poll();
  // Waiting restores start in block order and stop at the first the tier refuses: started ones stay a prefix of each
  // chain, and a full tier is asked once per poll, not once per waiting block (Cache::pollTransfers, Cache.cpp:938-956).
  bool refused = false, progressed = std::exchange(stateWriteRetired_, false);
  for (auto entry = restores_.begin(); entry != restores_.end();) {
    Transfer &t = entry->second;
    if (!t.ticket) {
      if (!refused && tier_->canRestore()) t.ticket = tier_->restore(t.slot, t.page);
      if (!t.ticket) refused = true;
      ++entry;
      continue;
    }
    if (!t.ticket->ready()) { ++entry; continue; }
    const bool landed = t.ticket->finish();
    index_.setTransferring(t.block, false);
    for (uint64_t waiter : t.waiters) {
      auto waiting = requests_.find(waiter);
      if (waiting == requests_.end()) continue;
      --waiting->second.pendingRestores;
      if (!landed) waiting->second.restoreFailed = true;
    }
    if (landed) {
      ++counters_.restoresLanded;
    } else {
      ++counters_.failedTransfers;
      states_.invalidate(t.block); // so does any state it held
      index_.poison(t.block);  // it matches nothing any more; its users recompute
      poisoned_.push_back(t.block);
    }
    entry = restores_.erase(entry);
    progressed = true;
  }
  // demotions after the restores, as the reference retires them (Cache.cpp:978-998): a waiting read starts at the
  // poll after the one that retired the write whose place it takes
  for (size_t i = 0; i < demotions_.size();) {
    Transfer &t = demotions_[i];
    if (!t.ticket->ready()) { ++i; continue; }
    const bool landed = t.ticket->finish();
    index_.setTransferring(t.block, false);
    if (landed) {
      ++counters_.demotionsLanded;
      index_.setSlot(t.block, t.slot);
      // a state published on the block while its copy was in flight keeps the page under it
      if (index_.residentLeaf(t.block) && !states_.stateResident(t.block)) { index_.dropPage(t.block); ++counters_.evictedBlocks; }
    } else {
      ++counters_.failedTransfers; // the page stays: a failed demotion loses nothing
    }
    demotions_.erase(demotions_.begin() + long(i));
    progressed = true;
  }
  if (progressed) dropPoisoned(); // only a transfer that retired can have freed what a poisoned block waited for
}

bool Cache::compactExtent() {
  std::vector<uint32_t> fixed; // pages a transfer reads or writes in place stay where they are
  for (const Transfer &t : demotions_) fixed.push_back(t.page);
  for (const auto &[block, t] : restores_) fixed.push_back(t.page);
  const KvPageMoves moves = pool_.compactExtent(fixed);
  if (moves.empty()) return false;
  index_.followPages(moves);
  for (auto &[id, active] : requests_) {
    uint32_t first = uint32_t(active.pages.size());
    for (uint32_t i = 0; i < active.pages.size(); ++i) {
      const uint32_t to = moves.follow(active.pages[i]);
      if (to != active.pages[i]) { active.pages[i] = to; first = std::min(first, i); }
    }
    if (first < active.pages.size()) changed(active, first);
  }
  return true;
}

CacheSnapshot Cache::snapshot() const {
  CacheSnapshot result = counters_;
  result.requests = uint32_t(requests_.size());
  result.residentBlocks = index_.residentBlocks();
  result.tierBlocks = index_.tierBlocks();
  result.transfers = uint32_t(demotions_.size() + restores_.size());
  result.pendingPages = pendingPages();
  return result;
}

// ============================== persistence ====================================================
uint32_t Cache::persist(model::SlotStore &store) {
  if (!tier_) throw std::logic_error("only a cache with a tier keeps copies");
  if (store.slotBytes() < tier_->slotBytes() || store.labelBytes() != sizeof(model::KvBlockLabel))
    throw std::invalid_argument("the slot store was opened for another kind of slot");
  // The new set is written beside the old one and flushed before the old one is freed: a crash or an IO error part
  // way leaves the previous seal whole (plus some records of the new one, which adopt() takes or drops one by one).
  // The new set goes below the old one when it fits there, else above it.
  const auto copies = index_.tierCopies();
  const std::set<uint32_t> previous = store.recorded();
  const uint32_t base = previous.empty() || *previous.begin() >= copies.size() ? 0 : *previous.rbegin() + 1;
  uint32_t written = 0;
  for (const auto &[label, slot] : copies) {
    KvTier::SlotPayload payload;
    if (!tier_->slotPayload(*slot, &payload)) continue;
    const auto *bytes = static_cast<const uint8_t *>(payload.bytes);
    const auto *raw = reinterpret_cast<const uint8_t *>(&label);
    if (!store.write(base + written, {bytes, size_t(payload.size)}, payload.checksum, {raw, sizeof(label)}))
      throw std::runtime_error("a slot write failed; the previous seal and the slots written so far keep their records");
    ++written;
  }
  if (!store.synchronize()) throw std::runtime_error("the slot store could not be flushed");
  for (uint32_t index : previous)
    if (!store.free(index)) throw std::runtime_error("a slot of the previous seal could not be freed");
  if (!store.synchronize()) throw std::runtime_error("the slot store could not be flushed");
  return written;
}

Cache::Adoption Cache::adopt(model::SlotStore &store) { return adoptRecords(store, nullptr); }
Cache::Adoption Cache::adoptRestorePoints(model::SlotStore &store, std::span<const PersistedState> states) { return adoptRecords(store, &states); }

Cache::Adoption Cache::adoptRecords(model::SlotStore &store, const std::span<const PersistedState> *states) {
  if (!tier_) throw std::logic_error("a cache takes back copies only from a tier");
  if (!requests_.empty() || index_.size() || states_.size()) throw std::logic_error("a cache takes back copies only before anything else is in it");
  if (store.labelBytes() != sizeof(model::KvBlockLabel)) throw std::invalid_argument("the slot store holds another kind of label");
  Adoption result;
  // tokens: up to and including the block by the labels alone; zero while its chain is broken.
  struct Recorded { model::KvBlockLabel label; const model::SlotRecord *record = nullptr; uint32_t tokens = 0; bool needed = false; };
  std::map<uint64_t, Recorded> recorded;
  uint64_t highestId = 0, lastUsed = 0;
  for (const model::SlotRecord &record : store.records()) {
    model::KvBlockLabel label;
    const bool sized = record.label.size() == sizeof(label);
    if (sized) {
      std::memcpy(&label, record.label.data(), sizeof(label));
      highestId = std::max(highestId, label.id);
    }
    if (!sized || !label.id || label.parent >= label.id || record.payloadBytes != tier_->slotBytes() ||
        !recorded.emplace(label.id, Recorded{label, &record}).second) {
      ++result.dropped;
      store.free(record.index);
    }
  }
  // A parent's id is lower than its children's, so a chain resolves in id order and a cycle cannot form.
  for (auto &[id, block] : recorded) {
    if (!block.label.parent) {
      block.tokens = PrefixIndex::pageTokens;
    } else if (auto parent = recorded.find(block.label.parent); parent != recorded.end() && parent->second.tokens) {
      block.tokens = parent->second.tokens + PrefixIndex::pageTokens;
    }
    block.needed = !states && block.tokens; // without the state layer every whole chain comes back
  }
  std::vector<const PersistedState *> kept;
  if (states) {
    for (const PersistedState &state : *states) {
      highestId = std::max(highestId, state.label.block);
      const auto block = recorded.find(state.label.block);
      if (block == recorded.end() || !block->second.tokens || block->second.tokens != state.label.tokens || !state.bytes) {
        ++result.dropped;
        continue;
      }
      kept.push_back(&state);
      for (auto above = block; above != recorded.end() && !above->second.needed; above = recorded.find(above->second.label.parent))
        above->second.needed = true;
    }
  }
  // A record whose payload cannot be read, or whose key another block took, stays behind, and so does everything below.
  std::vector<uint8_t> payload(tier_->slotBytes());
  std::set<uint64_t> adopted;
  for (auto &[id, block] : recorded) {
    bool taken = false;
    if (block.needed && (!block.label.parent || adopted.count(block.label.parent)) && store.read(block.record->index, payload)) {
      if (auto slot = tier_->adoptSlot(payload.data(), payload.size(), block.record->checksum))
        taken = index_.adoptTierBlock(id, block.label.parent, block.label.tokens, {block.label.imagesLo, block.label.imagesHi},
                                      std::move(slot), block.label.lastUsed);
    }
    if (!taken) {
      ++result.dropped;
      store.free(block.record->index);
      continue;
    }
    adopted.insert(id);
    lastUsed = std::max(lastUsed, block.label.lastUsed);
    ++result.blocks;
  }
  // A block holds one state; a second label for it is a stale one.
  uint64_t stateBytes = 0;
  for (const PersistedState *state : kept) {
    if (adopted.count(state->label.block) && !states_.contains(state->label.block)) {
      states_.adoptStored(state->label.block, state->bytes, state->label.lastUsed, state->label.checkpoint != 0);
      lastUsed = std::max(lastUsed, state->label.lastUsed);
      stateBytes += state->bytes;
      ++result.states;
    } else {
      ++result.dropped;
    }
  }
  // New ids continue after every id a record names, taken back or not.
  index_.continueAfter(highestId, lastUsed);
  result.bytes = stateBytes + uint64_t(result.blocks) * tier_->slotBytes();
  return result;
}

std::vector<Cache::PersistedState> Cache::stateLabels() const {
  std::vector<PersistedState> labels;
  for (const StateCache::StoredState &state : states_.storedStates()) {
    if (!index_.contains(state.block)) continue;
    uint32_t blocks = 0;
    for (uint64_t at = state.block; at; at = index_.parent(at)) ++blocks;
    labels.push_back({model::StateLabel{state.block, state.lastUsed, blocks * PrefixIndex::pageTokens, state.checkpoint ? 1u : 0u}, state.bytes});
  }
  return labels;
}

} // namespace rkb::engine
