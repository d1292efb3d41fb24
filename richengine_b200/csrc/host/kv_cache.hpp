// kv_cache.hpp — request page lists, prefix-page sharing and eviction over the pool.
//
// PrefixIndex is the content-addressed chain of 32-token blocks of the reference
// (runtime/engine/cache/KvCache.hpp:40-239, KvCache.cpp): key = (parent block, the page's 32
// token ids, image identity), hash h ^= v + 0x9e3779b97f4a7c15 + (h<<6) + (h>>2) seeded with
// 0x6a09e667f3bcc909, exact compare on a hit, one prefix reference per resident block.
// Cache is the request-facing subset of the reference facade (runtime/engine/cache/Cache.hpp:213-436,
// Cache.cpp:143-177,236-333,381-413,436-550,794-851,933-1021): page lists with revisions, ensureTokens,
// publishCommittedBlocks (dedupe onto the shared page), lookup / attach of a cached prefix, reclaim of
// the oldest idle leaf through the tier, transfer retirement. Two extensions BASELINE.json asks for that
// the reference does not have: forkRequest (share full pages, copy the partial tail page) and truncate
// (give back the pages past a rejected speculative tail). Also here: the coupling of composite recurrent states
// to KV blocks (policy only: a state's buffers are a byte count), image identity in a block's key, lookup probes,
// and sealing / adopting tier copies through the slot store. The recurrent-state buffers themselves and the
// reference's disk directory (CacheDirectory) are outside this path.
#pragma once

#include "kv_pool.hpp"
#include "kv_tier.hpp"
#include "slot_store.hpp"
#include "state_cache.hpp"

#include <functional>
#include <map>

#include <array>
#include <cstdint>
#include <memory>
#include <optional>
#include <set>
#include <span>
#include <unordered_map>
#include <vector>

namespace rkb::engine {

struct ImageIdentity final {
  uint64_t lo = 0, hi = 0;
  bool operator==(const ImageIdentity &) const = default;
};
// One image in a prompt (ImageSpan, runtime/model/Model.hpp:130-146): the run of placeholder tokens it occupies, the
// patch grid of its resized pixels and a 128-bit digest of that content. Placeholder token ids are the same for every
// image, so a block's key carries the identity of the images that overlap it. Spans are sorted and disjoint.
struct ImageSpan final {
  uint32_t offset = 0, tokens = 0, gridHeight = 0, gridWidth = 0;
  uint64_t digestLo = 0, digestHi = 0;
  uint32_t end() const noexcept { return offset + tokens; }
};
// The identity of the images that overlap tokens [blockBegin, blockBegin + blockTokens): zero for text alone; two
// independently seeded chains fold each overlapping span's digest, grid, placement and the block's own position
// (blockImageIdentity, runtime/engine/cache/KvCache.cpp:29-52).
ImageIdentity blockImageIdentity(uint64_t blockBegin, uint32_t blockTokens, std::span<const ImageSpan> spans) noexcept;

class PrefixIndex final {
public:
  static constexpr uint32_t pageTokens = kv::kPageTokens;
  static constexpr uint32_t noPage = 0xffffffffu;
  struct Match { uint64_t id = 0; uint32_t page = noPage; };
  struct Chain { std::vector<uint64_t> blocks; std::vector<uint32_t> pages; };
  struct Candidate { uint64_t block = 0; uint64_t lastUsed = 0; };

  explicit PrefixIndex(KvPool &pool) : pool_(pool), blockOnPage_(pool.pageCount()) {}
  ~PrefixIndex();
  PrefixIndex(const PrefixIndex &) = delete;
  PrefixIndex &operator=(const PrefixIndex &) = delete;

  std::optional<Match> find(uint64_t parent, std::span<const uint32_t> tokens, ImageIdentity images = {}) const;
  // Existing content is returned as is; a host-only block adopts the writer's page; a block in
  // transfer keeps its own page and the writer keeps its copy.
  Match insert(uint64_t parent, std::span<const uint32_t> tokens, uint32_t page, ImageIdentity images = {});
  void retainActive(uint64_t block);
  void releaseActive(uint64_t block) noexcept;
  void touch(uint64_t block) noexcept;
  Chain chain(uint64_t block) const;
  bool contains(uint64_t block) const noexcept { return blocks_.count(block) != 0; }
  // In the graph and not poisoned (KvCache::matchable, KvCache.cpp:279-282).
  bool matchable(uint64_t block) const noexcept { auto found = blocks_.find(block); return found != blocks_.end() && !found->second.poisoned; }
  // Moves with every new block, adopted record, poisoning and erase (KvCache::generation, KvCache.hpp:228-233): while
  // it stands still, every chain a probe matched still matches and nothing extends it. Blocks leave leaf first and a
  // poisoned block hides those below it, so after a change a probe's chain holds up to its first unmatchable block.
  uint64_t generation() const noexcept { return generation_; }
  uint32_t page(uint64_t block) const { return at(block).page; }
  uint64_t parent(uint64_t block) const { return at(block).parent; }
  std::shared_ptr<KvTierSlot> slot(uint64_t block) const { return at(block).slot; }
  bool transferring(uint64_t block) const { return at(block).transferring; }
  bool idle(uint64_t block) const { const Block &b = at(block); return !b.activeUsers && !b.transferring; }
  bool residentLeaf(uint64_t block) const { const Block &b = at(block); return b.page != noPage && !b.residentChildren && !b.activeUsers && !b.transferring && !b.poisoned; }
  uint64_t lastUsed(uint64_t block) const { return at(block).lastUsed; }
  void setTransferring(uint64_t block, bool value) { at(block).transferring = value; refresh(block); }
  // A block without a page is erased, not stripped of its only copy (KvCache::setSlot, KvCache.cpp:379-385).
  void setSlot(uint64_t block, std::shared_ptr<KvTierSlot> slot);
  // The oldest idle block whose tier copy can make room in a full tier (KvCache::diskCandidate, KvCache.cpp:486-492):
  // `duplicate` = a copy of a page that is resident too (dropping it loses nothing), else a tier-only block without
  // children (dropping it loses the block). `after` continues in (recency, id) order.
  std::optional<Candidate> tierCandidate(bool duplicate, const Candidate *after = nullptr) const;
  // Children that live only in the tier (KvCache::hasDiskChildren, KvCache.cpp:294-297).
  bool tierChildren(uint64_t block) const { const Block &b = at(block); return b.children > b.residentChildren; }
  // Everything below a block, children before parents; empty when a block below is in use or in transfer
  // (KvCache::subtree, KvCache.cpp:494-514).
  std::vector<uint64_t> subtree(uint64_t block) const;
  bool poisoned(uint64_t block) const { return at(block).poisoned; }
  // Returns the page of a resident leaf that has a tier copy to the pool.
  void dropPage(uint64_t block);
  // A restore that was never submitted is taken back: the page returns and the block is tier-only again. False when
  // a resident block below or a request depends on it (KvCache::abandonRestore, KvCache.cpp:411-418).
  bool abandonRestore(uint64_t block);
  // Gives a host-only block a page whose content follows (restore, or recomputation).
  void adoptPage(uint64_t block, uint32_t page);
  void followPages(const KvPageMoves &moves) noexcept;
  void poison(uint64_t block);
  void erase(uint64_t block); // only a block without children, users or transfer
  std::optional<Candidate> evictionCandidate() const; // oldest resident leaf no request uses
  // The oldest such leaf after `after` in (recency, id) order that `accept` takes (KvCache::evictionCandidate(after)).
  std::optional<Candidate> evictionCandidate(const Candidate *after, const std::function<bool(uint64_t)> &accept) const;
  // States on the blocks strictly below a block, all of them and those in use (KvCache::stateBelow,
  // KvCache::stateInUseBelow): a state at `block` appeared or went.
  void adjustStatesBelow(uint64_t block, int states, int inUse);
  bool stateBelow(uint64_t block) const { return at(block).statesBelow != 0; }
  bool stateInUseBelow(uint64_t block) const { return at(block).statesInUseBelow != 0; }
  uint32_t children(uint64_t block) const { return at(block).children; }
  // A reusable state was published at the block at some time (KvCache::noteState / hadState).
  void noteState(uint64_t block) { at(block).hadState = true; }
  bool hadState(uint64_t block) const { return at(block).hadState; }
  uint64_t tick() noexcept { return ++clock_; }
  // Takes back a tier-only block an earlier process recorded (KvCache::adoptDiskBlock,
  // runtime/engine/cache/KvCache.cpp:160-199): false when another block already holds its key.
  bool adoptTierBlock(uint64_t id, uint64_t parent, std::span<const uint32_t> tokens, ImageIdentity images,
                      std::shared_ptr<KvTierSlot> slot, uint64_t lastUsed);
  // New ids and recency continue after everything a record names.
  void continueAfter(uint64_t highestId, uint64_t lastUsed) noexcept;
  // Every block whose tier copy has landed, in id order, as its record's label.
  std::vector<std::pair<model::KvBlockLabel, std::shared_ptr<KvTierSlot>>> tierCopies() const;
  uint32_t residentBlocks() const noexcept { return resident_; }
  uint32_t tierBlocks() const noexcept;
  size_t size() const noexcept { return blocks_.size(); }

private:
  struct Block {
    uint64_t id = 0, parent = 0, hash = 0, lastUsed = 0;
    std::array<uint32_t, pageTokens> tokens{};
    ImageIdentity images;
    uint32_t page = noPage;
    std::shared_ptr<KvTierSlot> slot;
    uint32_t children = 0, residentChildren = 0, activeUsers = 0;
    uint32_t statesBelow = 0, statesInUseBelow = 0;
    bool transferring = false, poisoned = false, hadState = false;
    bool listed = false;   // in idleLeaves_ under (listedAt, id)
    uint64_t listedAt = 0;
    uint8_t tierListed = 0; // 1 = in duplicates_, 2 = in tierLeaves_, under (tierListedAt, id)
    uint64_t tierListedAt = 0;
  };
  // Keeps idleLeaves_ in step with a block whose page, children, users, transfer or recency changed.
  void refresh(uint64_t block);
  static void inherit(Block &parent, uint64_t lastUsed) noexcept;
  // A poisoned block leaves as soon as nothing hangs on it: no child, no user, no transfer (KvCache::erasePoisonedLeaf).
  void erasePoisonedLeaf(uint64_t block) noexcept;
  Block &at(uint64_t block);
  const Block &at(uint64_t block) const;

  KvPool &pool_;
  std::unordered_map<uint64_t, Block> blocks_;
  std::unordered_multimap<uint64_t, uint64_t> index_;
  std::vector<uint64_t> blockOnPage_;
  // The resident leaves no request uses and no transfer touches, oldest first: the order evictions go in. Kept
  // current by every mutator, so a candidate costs a tree step instead of a pass over every block.
  std::set<std::pair<uint64_t, uint64_t>> idleLeaves_; // (last used, id)
  // Idle blocks with a tier copy, oldest first: copies of resident pages, and tier-only blocks without children.
  std::set<std::pair<uint64_t, uint64_t>> duplicates_, tierLeaves_;
  uint64_t nextId_ = 1, clock_ = 0, generation_ = 1;
  uint32_t resident_ = 0;
};

enum class TokenAdmissionFailure : uint8_t { None, Denied, Pending };
struct TokenAdmission {
  TokenAdmissionFailure failure = TokenAdmissionFailure::None;
  uint32_t pagesNeeded = 0, pagesFree = 0;
  AllocationFailure cause = AllocationFailure::None;
  bool granted() const noexcept { return failure == TokenAdmissionFailure::None; }
};

// A request's logical page list as the GPU table sees it: equal to the previous revision's below
// firstChanged (Cache.hpp:136-140; runtime/model/RuntimeBindings.hpp:205-233 patches from there).
struct PageTableView {
  std::span<const uint32_t> pages;
  uint64_t revision = 0;
  uint32_t firstChanged = 0;
};

struct CacheSnapshot {
  uint32_t requests = 0, residentBlocks = 0, tierBlocks = 0, transfers = 0;
  uint64_t demotions = 0, restores = 0, failedTransfers = 0, evictedBlocks = 0, forkCopies = 0, truncatedPages = 0;
  uint64_t demotionsRefused = 0, replacedCopies = 0, cancelledRestores = 0;
  uint64_t demotionsLanded = 0, restoresLanded = 0; // as the reference counts them (KvTierSnapshot::demotions / restores)
  uint32_t pendingPages = 0;
};

// How far a reclaim may reach (Cache.hpp: ReclaimClass): states in use, and the KV they restore through, go only to
// running work.
enum class ReclaimClass : uint8_t { Ordinary, InUse };
struct ReclaimStep { bool madeProgress = false, pending = false, evictedState = false; uint64_t reclaimedBytes = 0; };

class Cache final {
public:
  Cache(KvPool &pool, kv::ExtentStorage &storage, KvTier *tier = nullptr)
      : pool_(pool), storage_(storage), tier_(tier), index_(pool),
        states_([this](uint64_t block, int states, int inUse) { if (index_.contains(block)) index_.adjustStatesBelow(block, states, inUse); },
                [this] { return index_.tick(); },
                [this](uint64_t block) { if (index_.contains(block)) index_.noteState(block); },
                [this](uint64_t block, bool held) {
                  if (!index_.contains(block)) return;
                  if (held) index_.retainActive(block); else index_.releaseActive(block);
                }) {}
  ~Cache();

  // ---- composite states and the reclaim order they impose (runtime/engine/cache/Cache.cpp:451-628) ----------------
  StateCache &states() noexcept { return states_; }
  const StateCache &states() const noexcept { return states_; }
  // A complete block of a request's chain (Cache::blockAt): the block that ends at `tokens`, 0 when not published.
  uint64_t blockAt(uint64_t request, uint32_t tokens) const;
  void publishCompositeState(uint64_t block, uint64_t bytes, bool checkpoint);
  // A state the model stores elsewhere (StateCache::publishStored). Its write counts as retired at the next poll,
  // which therefore looks at the poisoned blocks again, as the reference's does after a state write (Cache.cpp:933-934).
  void publishStoredState(uint64_t block, uint64_t bytes, bool checkpoint);
  // Only a state restores a chain that has left the pool, through its own block and every block above
  // (Cache.hpp:549-556): such KV is needed by that state, and in use when the state is.
  bool kvNeededByState(uint64_t block) const { return states_.contains(block) || index_.stateBelow(block); }
  bool kvNeededByStateInUse(uint64_t block) const { return (states_.inUse(block) && states_.contains(block)) || index_.stateInUseBelow(block); }
  // One step of eviction in the reference's order (Cache::evictOne, Cache::reclaimOldest): disposable checkpoints
  // first (not in a page scan); then KV leaves no state needs, oldest first; then ordinary states and the leaves
  // under them by shared recency (a leaf gives up the state on it first); states in use and the KV they need
  // last, only up to ReclaimClass::InUse and once no transfer in flight can return what is needed.
  ReclaimStep evictOne(ReclaimClass upTo, bool keepResumePoint, bool pagesOnly);
  // Room for one more state (Cache::reclaimOneState): a checkpoint; unless checkpointsOnly an ordinary state; a state
  // in use only for a publication that is itself in use (forBlock).
  bool reclaimOneState(bool checkpointsOnly, uint64_t forBlock);

  void beginRequest(uint64_t request);
  void endRequest(uint64_t request);
  TokenAdmission ensureTokens(uint64_t request, uint64_t tokenCount);
  PageTableView pageTable(uint64_t request) const;
  // Hashes each newly complete page into the index; content that already exists swaps the request onto
  // the shared page and releases the writer's copy (Cache.cpp:294-333).
  void publishCommittedBlocks(uint64_t request, std::span<const uint32_t> exactTokens, uint32_t committedTokens,
                              std::span<const ImageSpan> images = {});
  // The cached chain matching the prompt: at most (n-1)/32 blocks, one real token is always left
  // to recompute (Cache.cpp:179-199).
  struct Probe;
  std::vector<uint64_t> lookup(std::span<const uint32_t> prompt, const Probe *probe = nullptr, std::span<const ImageSpan> images = {});
  // The lookup a hybrid model's admission makes (Cache::lookup, Cache.cpp:236-272; CacheLookup, Cache.hpp:20-36):
  // the matched chain, the deepest state on it (pinned for the caller, as the reference's lease pins it: unpin with
  // states().unpin(stateBlock) once the restore is done), where the request resumes, whether the matched KV ends at
  // a branch point past the state with another branch's state below it (a junction worth materialising a state
  // at), and whether a matched block past the state once held a reusable state that is gone.
  struct StateLookup {
    std::vector<uint64_t> blocks;
    uint32_t kvBoundary = 0, resumeBoundary = 0, junctionBoundary = 0;
    uint64_t stateBlock = 0;
    bool lostState = false;
  };
  // What a scheduler keeps per waiting request between admission passes (CacheProbe, Cache.hpp:38-52; Cache::probe,
  // Cache::refresh, Cache.cpp:210-234): the matched chain, the generation of the block graph it was matched under and
  // the tokens up to the deepest state on it. A probe pins nothing, touches no recency and counts no hit. While the
  // graph's generation stands still a refresh hashes nothing (states come and go without it, so the cached tokens
  // are always looked up again); after a change the chain is cut at its first unmatchable block and only the pages
  // past the cut are hashed. A lookup given a current probe of this cache reuses its chain; a stale or foreign probe
  // is ignored there and a foreign one is refused by refresh.
  struct Probe {
    uint32_t cachedTokens() const noexcept { return cachedTokens_; }
    const std::vector<uint64_t> &blocks() const noexcept { return blocks_; }
   private:
    friend class Cache;
    std::vector<uint64_t> blocks_;
    uint64_t generation_ = 0;
    uint32_t cachedTokens_ = 0;
    const Cache *owner_ = nullptr;
  };
  Probe probe(std::span<const uint32_t> prompt, std::span<const ImageSpan> images = {});
  void refresh(Probe &probe, std::span<const uint32_t> prompt, std::span<const ImageSpan> images = {});
  StateLookup lookupWithState(std::span<const uint32_t> prompt, const Probe *probe = nullptr, std::span<const ImageSpan> images = {});
  // Counts a lookup that admission acted on (Cache::recordLookup, Cache.cpp:274-282); probeHashedBlocks counts the
  // pages probes hashed (CacheLookupSnapshot::probeHashedBlocks).
  struct LookupCounters { uint64_t kvHitTokens = 0, lazyJunctions = 0, lostStateMisses = 0, probeHashedBlocks = 0; };
  void recordLookup(const StateLookup &lookup) noexcept;
  LookupCounters lookupCounters() const noexcept { return lookups_; }
  // Attaches a matched chain to a request without pages: resident blocks are shared (one more
  // active reference each), host-only blocks take fresh pages and start restores, root first
  // (Cache.cpp:745-785). Returns the tokens the request resumes after, or Denied/Pending.
  TokenAdmission attachPrefix(uint64_t request, std::span<const uint64_t> blocks, uint32_t *resumeTokens);
  bool restoresPending(uint64_t request) const;
  int restoreStatus(uint64_t request) const;

  // Extension: `child` shares every full committed page of `parent` and gets its own copy of the
  // partial tail page (copy-on-write of the only page both would write). Copies are ordered on the
  // storage's stream. Returns the number of pages copied (0 or 1), or throws on refusal.
  uint32_t forkRequest(uint64_t parent, uint64_t child, uint32_t committedTokens);
  // Extension: after a verify step committed `committedTokens`, keep the pages that hold them plus
  // `scratchTokens` ahead and give the rest back. Returns the pages released.
  uint32_t truncate(uint64_t request, uint32_t committedTokens, uint32_t scratchTokens);

  // Evicts the oldest idle leaf: with a tier, starts its demotion (the page stays until the copy
  // lands); without one, or when the block already has a tier copy, drops it at once.
  bool reclaimOne();
  uint32_t reclaimForPages(uint32_t pages);
  // One step of making room, as the reference's governor asks for it (Cache::reclaimOne with CacheReclaimMode,
  // Cache.cpp:436-449, releaseExtent :692-698): memory returns as whole extents. ReleaseExtents: an empty extent goes
  // as it is; else the free pages scattered over the others are gathered until they fill one (compactExtent) and that
  // one goes; else one victim is evicted (and the extent it may have emptied goes with it). KeepExtents only evicts;
  // ReusePages evicts in a page scan (a state's buffers give no page). keepRunway leaves the one empty extent a pass
  // keeps. reclaimedBytes counts the bytes of the extents returned to the device (a step that evicts a state says so
  // in evictedState; its buffers go back to the model's pool).
  enum class ReclaimMode : uint8_t { ReleaseExtents, KeepExtents, ReusePages };
  ReclaimStep reclaimStep(ReclaimMode mode, ReclaimClass upTo, bool keepResumePoint = false, bool keepRunway = false);
  // Everything unpinned goes before anything moves, then every extent that can be emptied is (Cache::evictAll,
  // Cache.cpp:423-434).
  ReclaimStep evictAll();
  uint64_t releaseEmptyExtents(bool keepRunway) { return pool_.reclaimEmptyExtents(keepRunway, 0xffffffffu); }
  // Retires finished transfers (Cache.cpp:933-1021): a landed demotion drops the page, a failed one
  // keeps it; a landed restore makes the block usable, a failed one poisons it.
  void pollTransfers();
  // Empties one extent (KvPool::compactExtent) and re-points every request and block.
  bool compactExtent();
  uint32_t pendingPages() const noexcept { return uint32_t(demotions_.size()); }
  // A hybrid model resumes a chain only through a composite state: KV no state needs is then not worth a tier copy
  // and is dropped instead of written, as the reference does (Cache::reclaimKvLeaf, Cache.cpp:629-659). Off (the
  // default) every block is worth its copy: an attention-only model resumes from KV alone.
  void setStateCoupled(bool coupled) noexcept { stateCoupled_ = coupled; }

  // Seals every landed tier copy into the store with its label (the record Cache::labelBlock keeps,
  // runtime/engine/cache/Cache.cpp:852-870): payload, CRC-32C, KvBlockLabel. The store is rewritten whole and
  // flushed. Returns the slots written.
  uint32_t persist(model::SlotStore &store);
  // Before anything else is in the cache: takes back the blocks an earlier process sealed (Cache::adopt,
  // runtime/engine/cache/Cache.cpp:38-140): labels resolve in id order (a parent's id is lower than its
  // children's), a block comes back only under an unbroken chain, a duplicate key or a damaged label stays
  // behind, and the records that stay behind are freed. A payload is checked against its record's CRC-32C when
  // it is first restored. Without the reference's composite-state layer every intact chain comes back.
  struct Adoption { uint32_t blocks = 0, dropped = 0; uint64_t bytes = 0; uint32_t states = 0; };
  Adoption adopt(model::SlotStore &store);
  // The reference's rule for a cache whose chains resume only through composite states (Cache::adopt,
  // runtime/engine/cache/Cache.cpp:70-127): a state comes back with its whole chain, stored; a block only for a state.
  // A state whose block has no whole chain, or whose label names another boundary than the chain's length, stays
  // behind, and so does a second state of one block; `dropped` counts those too. Ids continue after every id a block
  // or state label names.
  struct PersistedState { model::StateLabel label; uint64_t bytes = 0; };
  Adoption adoptRestorePoints(model::SlotStore &store, std::span<const PersistedState> states);
  // The label of every stored state as a clean stop writes it (Cache::relabelStates, StateCache::labelDisk): block,
  // recency, the chain's length in tokens, class.
  std::vector<PersistedState> stateLabels() const;

  PrefixIndex &index() noexcept { return index_; }
  CacheSnapshot snapshot() const;

private:
  Adoption adoptRecords(model::SlotStore &store, const std::span<const PersistedState> *states);
  struct Request {
    std::vector<uint32_t> pages;
    std::vector<uint64_t> blocks; // cached chain covering the first blocks.size() pages
    uint64_t revision = 0;
    uint32_t firstChanged = 0;
    uint32_t pendingRestores = 0; // reads this request attached to and waits for (Cache::restoreRequest's waiters)
    bool restoreFailed = false;
  };
  struct Transfer {
    uint64_t block = 0;
    uint32_t page = 0;
    std::unique_ptr<KvTransfer> ticket;
    std::shared_ptr<KvTierSlot> slot;
    std::vector<uint64_t> waiters; // the requests that attached to a read
  };
  enum class LeafReclaim : uint8_t { Started, Pending, Impossible };
  LeafReclaim reclaimKvLeaf(uint64_t block, bool immediate = false);
  LeafReclaim demoteKv(uint64_t block);
  std::shared_ptr<KvTierSlot> acquireTierSlot(bool inUse);
  bool freeTierSpace(bool inUse);
  bool dropTierSubtree(uint64_t block);
  ReclaimStep releaseExtent(bool keepRunway);
  void dropPoisoned();
  bool tierWritable() const noexcept { return tier_ && tier_->writable(); }
  bool worthACopy(uint64_t block) const { return !stateCoupled_ || kvNeededByState(block); }
  struct Victim { bool kv = false; };
  std::optional<Victim> reclaimOldest(bool inUse, bool keepResumePoint, bool pagesOnly);
  bool transfersInFlight() const noexcept { return !demotions_.empty() || !restores_.empty(); }
  Request &request(uint64_t id);
  const Request &request(uint64_t id) const;
  static void changed(Request &r, uint32_t first) noexcept { ++r.revision; r.firstChanged = first; }
  TokenAdmission admitPages(uint32_t count, std::vector<uint32_t> &pages);

  KvPool &pool_;
  kv::ExtentStorage &storage_;
  KvTier *tier_;
  PrefixIndex index_;
  StateCache states_;
  LookupCounters lookups_;
  size_t extendMatch(std::vector<uint64_t> &blocks, std::span<const uint32_t> prompt, std::span<const ImageSpan> images) const;
  uint32_t stateTokens(std::span<const uint64_t> blocks) const;
  std::unordered_map<uint64_t, Request> requests_;
  std::vector<Transfer> demotions_;
  std::map<uint64_t, Transfer> restores_; // by block: a parent's id is lower than its children's, so this is chain order
  std::vector<uint64_t> poisoned_; // blocks whose restore failed, until they and what hangs below them have gone
  bool stateCoupled_ = false, stateWriteRetired_ = false;
  CacheSnapshot counters_;
};

} // namespace rkb::engine
