// host_capi.cpp — C handles over the host control plane (include/richkv_host.h).
#include "../../../include/richkv_host.h"

#include "kv_cache.hpp"
#include "kv_pool.hpp"
#include "paged_attention.hpp"
#include "storage_adapters.hpp"

#include <cuda_runtime.h>

#include <cstring>
#include <deque>
#include <memory>
#include <stdexcept>
#include <string>

namespace rk { void set_error(const char *text); }

using namespace rkb;

namespace {

struct PoolHandle {
  std::unique_ptr<kv::BudgetExtentStorage> budget;
  std::unique_ptr<kv::DeviceExtentStorage> device;
  std::unique_ptr<engine::KvPool> pool;
  kv::ExtentStorage &storage() { return budget ? static_cast<kv::ExtentStorage &>(*budget) : *device; }
};

// A tier without a device: slots hold content tags; transfers finish when the test says so
// (the shape of the reference's test tier, dev/tests/engine/TestKvTier.hpp:17-127).
class ManualTier final : public engine::KvTier {
public:
  ManualTier(kv::BudgetExtentStorage &storage, uint32_t slots, uint32_t transfers)
      : storage_(storage), used_(slots, 0), tags_(slots, 0), expected_(slots, 0), arrived_(slots, 0), verify_(slots, 0),
        payloads_(slots), limit_(transfers) {}
  uint64_t slotBytes() const noexcept override { return storage_.bytesPerPage(); }
  bool writable() const noexcept override { return writable_; }
  // The shares of the pinned-host tier (demotions at most half, restores at most three quarters of the transfers in
  // flight), or, with plain limits, one bound on both kinds together as the reference's test tier has it
  // (dev/tests/engine/TestKvTier.hpp:35-36).
  // A transfer holds its place until the cache has retired it (KvTransfer::finish), not only until it has landed.
  bool canDemote() const noexcept override { return (plain_ || demotions_ < std::max(1u, limit_ / 2)) && inFlight_ < limit_ && writable_; }
  bool canRestore() const noexcept override { return (plain_ || restores_ < std::max(1u, limit_ - limit_ / 4)) && inFlight_ < limit_; }
  std::shared_ptr<engine::KvTierSlot> acquireSlot() override {
    for (uint32_t i = 0; i < used_.size(); ++i)
      if (!used_[i]) { used_[i] = 1; return std::make_shared<Slot>(this, i); }
    return {};
  }
  std::unique_ptr<engine::KvTransfer> demote(uint32_t page, std::shared_ptr<engine::KvTierSlot> slot) override {
    if (!canDemote()) return {};
    auto state = std::make_shared<State>(State{true, page, std::dynamic_pointer_cast<Slot>(slot)->id});
    pending_.push_back(state);
    ++demotions_; ++inFlight_;
    return std::make_unique<Ticket>(this, state);
  }
  std::unique_ptr<engine::KvTransfer> restore(std::shared_ptr<engine::KvTierSlot> slot, uint32_t page) override {
    if (!canRestore()) return {};
    auto state = std::make_shared<State>(State{false, page, std::dynamic_pointer_cast<Slot>(slot)->id});
    pending_.push_back(state);
    ++restores_; ++inFlight_;
    return std::make_unique<Ticket>(this, state);
  }
  void poll() override {}
  // A slot's payload is its content tag repeated over the slot, so that a slot store sees real bytes.
  bool slotPayload(const engine::KvTierSlot &slot, SlotPayload *out) const override {
    const auto *held = dynamic_cast<const Slot *>(&slot);
    if (!held) return false;
    std::vector<uint8_t> &bytes = payloads_[held->id];
    bytes.resize(slotBytes());
    for (size_t at = 0; at < bytes.size(); at += 8) std::memcpy(bytes.data() + at, &tags_[held->id], std::min<size_t>(8, bytes.size() - at));
    *out = {bytes.data(), bytes.size(), rk_crc32c_host(bytes.data(), bytes.size(), 0)};
    return true;
  }
  std::shared_ptr<engine::KvTierSlot> adoptSlot(const void *payload, uint64_t bytes, uint32_t checksum) override {
    if (bytes != slotBytes()) throw std::invalid_argument("the payload is not one slot");
    auto slot = std::dynamic_pointer_cast<Slot>(acquireSlot());
    if (!slot) return {};
    std::memcpy(&tags_[slot->id], payload, std::min<uint64_t>(8, bytes));
    expected_[slot->id] = checksum;
    arrived_[slot->id] = rk_crc32c_host(payload, bytes, 0);
    verify_[slot->id] = 1;
    return slot;
  }
  void set(uint32_t limit, bool writable) noexcept { limit_ = limit; writable_ = writable; }
  void setPlainLimits(bool plain) noexcept { plain_ = plain; }
  bool complete(bool success) {
    if (pending_.empty()) return false;
    auto state = pending_.front();
    pending_.pop_front();
    if (success && !state->demotion && verify_[state->slot]) { // an adopted slot's first read is checked against its record
      if (arrived_[state->slot] != expected_[state->slot]) success = false;
      else verify_[state->slot] = 0;
    }
    if (success) {
      if (state->demotion) tags_[state->slot] = storage_.content.at(state->page);
      else storage_.content.at(state->page) = tags_[state->slot];
    } else if (state->demotion && !plain_) {
      writable_ = false; // a failed write closes the tier (the test tier with plain limits stays as the test set it)
    }
    state->ready = true;
    state->success = success;
    return true;
  }

private:
  struct State { bool demotion; uint32_t page, slot; bool ready = false, success = false, retired = false; };
  struct Slot final : engine::KvTierSlot {
    Slot(ManualTier *t, uint32_t i) : tier(t), id(i) {}
    ~Slot() override { tier->used_[id] = 0; tier->verify_[id] = 0; }
    ManualTier *tier; uint32_t id;
  };
  struct Ticket final : engine::KvTransfer {
    Ticket(ManualTier *t, std::shared_ptr<State> s) : tier(t), state(std::move(s)) {}
    bool ready() const noexcept override { return state->ready; }
    bool finish() override {
      if (!state->retired) {
        state->retired = true;
        --tier->inFlight_;
        --(state->demotion ? tier->demotions_ : tier->restores_);
      }
      return state->success;
    }
    ManualTier *tier;
    std::shared_ptr<State> state;
  };
  kv::BudgetExtentStorage &storage_;
  std::vector<uint8_t> used_;
  std::vector<uint64_t> tags_;
  std::vector<uint32_t> expected_, arrived_;
  std::vector<uint8_t> verify_;
  mutable std::vector<std::vector<uint8_t>> payloads_;
  std::deque<std::shared_ptr<State>> pending_;
  uint32_t limit_, demotions_ = 0, restores_ = 0, inFlight_ = 0;
  bool writable_ = true, plain_ = false;
};

struct CacheHandle {
  PoolHandle *pool = nullptr;
  std::unique_ptr<engine::KvTier> tier;
  ManualTier *manual = nullptr;
  engine::HostKvTier *host = nullptr;
  std::unique_ptr<engine::Cache> cache;
};

template <typename F> int guarded(F &&body) {
  try {
    return body();
  } catch (const std::invalid_argument &e) { rk::set_error(e.what()); return RK_ERR_INVALID;
  } catch (const std::logic_error &e) { rk::set_error(e.what()); return RK_ERR_INVALID;
  } catch (const std::exception &e) { rk::set_error(e.what()); return RK_ERR_REFUSED; }
}

kv::Layout layoutOf(uint32_t layers, uint32_t heads, uint32_t dim, uint32_t format) {
  return kv::Layout{layers, heads, dim, static_cast<kv::Format>(format), 0.0f};
}
int joinNames(std::initializer_list<std::string> parts, char *names, size_t bytes) {
  std::string joined;
  for (const std::string &p : parts) { if (!joined.empty()) joined += "\n"; joined += p; }
  if (joined.size() + 1 > bytes) return RK_ERR_INVALID;
  std::memcpy(names, joined.c_str(), joined.size() + 1);
  return RK_OK;
}

} // namespace

extern "C" {

void *rk_pool_create_budget(uint32_t pages, uint64_t bytes_per_page, uint32_t extent_pages, uint32_t runway_pages, uint64_t budget_pages) {
  try {
    if (!extent_pages || !pages || pages % extent_pages) throw std::invalid_argument("invalid KV extent storage");
    auto h = std::make_unique<PoolHandle>();
    h->budget = std::make_unique<kv::BudgetExtentStorage>(pages, bytes_per_page, extent_pages);
    h->budget->budgetPages = budget_pages;
    h->pool = std::make_unique<engine::KvPool>(*h->budget, runway_pages);
    return h.release();
  } catch (const std::exception &e) { rk::set_error(e.what()); return nullptr; }
}
void *rk_pool_create_device(void *storage, uint32_t runway_pages, void *stream) {
  try {
    auto h = std::make_unique<PoolHandle>();
    h->device = std::make_unique<kv::DeviceExtentStorage>(storage, stream);
    h->pool = std::make_unique<engine::KvPool>(*h->device, runway_pages);
    return h.release();
  } catch (const std::exception &e) { rk::set_error(e.what()); return nullptr; }
}
void rk_pool_destroy(void *pool) { delete static_cast<PoolHandle *>(pool); }
void rk_pool_set_budget(void *pool, uint64_t budget_pages) {
  auto *h = static_cast<PoolHandle *>(pool);
  if (h->budget) h->budget->budgetPages = budget_pages;
}
int rk_pool_acquire(void *pool, uint32_t count, uint32_t *pages_out) {
  return guarded([&] {
    auto got = static_cast<PoolHandle *>(pool)->pool->acquirePages(count);
    if (!got.granted()) { rk::set_error("the pool could not grow by an extent"); return RK_ERR_REFUSED; }
    std::copy(got.pages.begin(), got.pages.end(), pages_out);
    return int(got.pages.size());
  });
}
int rk_pool_retain(void *pool, uint32_t page, int prefix_owner) {
  return guarded([&] { static_cast<PoolHandle *>(pool)->pool->retainPage(page, prefix_owner != 0); return RK_OK; });
}
int rk_pool_release(void *pool, uint32_t page, int prefix_owner) {
  return guarded([&] { static_cast<PoolHandle *>(pool)->pool->releasePage(page, prefix_owner != 0); return RK_OK; });
}
uint64_t rk_pool_reclaim_empty_extents(void *pool, int keep_runway, uint32_t limit) {
  return static_cast<PoolHandle *>(pool)->pool->reclaimEmptyExtents(keep_runway != 0, limit);
}
int64_t rk_pool_compact_extent(void *pool, const uint32_t *fixed, uint32_t fixed_count, uint32_t *destinations_out) {
  try {
    auto moves = static_cast<PoolHandle *>(pool)->pool->compactExtent({fixed, fixed_count});
    if (moves.empty()) return -1;
    std::copy(moves.destinations.begin(), moves.destinations.end(), destinations_out);
    return moves.firstPage;
  } catch (const std::exception &e) { rk::set_error(e.what()); return -2; }
}
void rk_pool_snapshot(const void *pool, uint64_t *out) {
  const auto s = static_cast<const PoolHandle *>(pool)->pool->snapshot();
  out[0] = s.pagesAllocated; out[1] = s.pagesFree; out[2] = s.pagesActive; out[3] = s.pagesPrefix;
  out[4] = s.allocatedBytes; out[5] = s.reclaimableBytes; out[6] = s.extentAllocations;
  out[7] = s.extentReleases; out[8] = s.extentCompactions; out[9] = s.pagesMoved;
}
uint64_t rk_pool_page_content(const void *pool, uint32_t page) {
  const auto *h = static_cast<const PoolHandle *>(pool);
  return h->budget ? h->budget->content.at(page) : 0;
}
void rk_pool_set_page_content(void *pool, uint32_t page, uint64_t tag) {
  auto *h = static_cast<PoolHandle *>(pool);
  if (h->budget) h->budget->content.at(page) = tag;
}

void *rk_cache_create(void *pool, int tier_mode, uint32_t slots, uint32_t transfers) {
  try {
    auto *p = static_cast<PoolHandle *>(pool);
    auto h = std::make_unique<CacheHandle>();
    h->pool = p;
    if (tier_mode == 1) {
      if (!p->device) throw std::invalid_argument("the pinned-host tier needs a device pool");
      auto tier = std::make_unique<engine::HostKvTier>(p->device->handle(), slots, transfers);
      h->host = tier.get();
      h->tier = std::move(tier);
    } else if (tier_mode == 2) {
      if (!p->budget) throw std::invalid_argument("the manual tier needs a budget pool");
      auto tier = std::make_unique<ManualTier>(*p->budget, slots, transfers);
      h->manual = tier.get();
      h->tier = std::move(tier);
    }
    h->cache = std::make_unique<engine::Cache>(*p->pool, p->storage(), h->tier.get());
    return h.release();
  } catch (const std::exception &e) { rk::set_error(e.what()); return nullptr; }
}
void rk_cache_destroy(void *cache) {
  auto *h = static_cast<CacheHandle *>(cache);
  if (!h) return;
  if (h->manual) while (h->manual->complete(true)) {} // nothing stays in flight
  h->cache.reset();
  delete h;
}
#define CACHE (static_cast<CacheHandle *>(cache)->cache)
int rk_cache_begin_request(void *cache, uint64_t request) { return guarded([&] { CACHE->beginRequest(request); return RK_OK; }); }
int rk_cache_end_request(void *cache, uint64_t request) { return guarded([&] { CACHE->endRequest(request); return RK_OK; }); }
int rk_cache_ensure_tokens(void *cache, uint64_t request, uint64_t tokens) {
  return guarded([&] { return int(CACHE->ensureTokens(request, tokens).failure); });
}
int64_t rk_cache_page_table(const void *cache, uint64_t request, uint32_t *pages_out, uint32_t capacity, uint64_t *revision, uint32_t *first_changed) {
  try {
    const auto view = static_cast<const CacheHandle *>(cache)->cache->pageTable(request);
    for (size_t i = 0; i < view.pages.size() && i < capacity; ++i) pages_out[i] = view.pages[i];
    if (revision) *revision = view.revision;
    if (first_changed) *first_changed = view.firstChanged;
    return int64_t(view.pages.size());
  } catch (const std::exception &e) { rk::set_error(e.what()); return RK_ERR_INVALID; }
}
// rk_image_span and engine::ImageSpan are the same 32 bytes.
static std::span<const engine::ImageSpan> image_spans(const rk_image_span *images, uint32_t count) {
  static_assert(sizeof(rk_image_span) == sizeof(engine::ImageSpan) && sizeof(rk_image_span) == 32);
  return {reinterpret_cast<const engine::ImageSpan *>(images), images ? count : 0u};
}
// blockImageIdentity: out[2] = lo, hi
void rk_block_image_identity(uint64_t block_begin, uint32_t block_tokens, const rk_image_span *images, uint32_t image_count, uint64_t *out) {
  const engine::ImageIdentity identity = engine::blockImageIdentity(block_begin, block_tokens, image_spans(images, image_count));
  out[0] = identity.lo; out[1] = identity.hi;
}
int rk_cache_publish(void *cache, uint64_t request, const uint32_t *tokens, uint32_t token_count, uint32_t committed,
                     const rk_image_span *images, uint32_t image_count) {
  return guarded([&] { CACHE->publishCommittedBlocks(request, {tokens, token_count}, committed, image_spans(images, image_count)); return RK_OK; });
}
int64_t rk_cache_lookup(void *cache, const uint32_t *prompt, uint32_t prompt_tokens, uint64_t *blocks_out, uint32_t capacity,
                        const rk_image_span *images, uint32_t image_count) {
  try {
    const auto blocks = CACHE->lookup({prompt, prompt_tokens}, nullptr, image_spans(images, image_count));
    for (size_t i = 0; i < blocks.size() && i < capacity; ++i) blocks_out[i] = blocks[i];
    return int64_t(blocks.size());
  } catch (const std::exception &e) { rk::set_error(e.what()); return RK_ERR_INVALID; }
}
int rk_cache_attach_prefix(void *cache, uint64_t request, const uint64_t *blocks, uint32_t count, uint32_t *resume_tokens) {
  return guarded([&] { return int(CACHE->attachPrefix(request, {blocks, count}, resume_tokens).failure); });
}
int rk_cache_restores_pending(const void *cache, uint64_t request) {
  try { return static_cast<const CacheHandle *>(cache)->cache->restoresPending(request) ? 1 : 0; } catch (...) { return RK_ERR_INVALID; }
}
int rk_cache_restore_status(const void *cache, uint64_t request) {
  try { return static_cast<const CacheHandle *>(cache)->cache->restoreStatus(request); } catch (...) { return RK_ERR_INVALID; }
}
void rk_cache_set_state_coupled(void *cache, int coupled) { CACHE->setStateCoupled(coupled != 0); }
int rk_cache_fork(void *cache, uint64_t parent, uint64_t child, uint32_t committed_tokens) {
  return guarded([&] { return int(CACHE->forkRequest(parent, child, committed_tokens)); });
}
int64_t rk_cache_truncate(void *cache, uint64_t request, uint32_t committed_tokens, uint32_t scratch_tokens) {
  try { return CACHE->truncate(request, committed_tokens, scratch_tokens); } catch (const std::exception &e) { rk::set_error(e.what()); return RK_ERR_INVALID; }
}
int rk_cache_reclaim_one(void *cache) { return guarded([&] { return CACHE->reclaimOne() ? 1 : 0; }); }
uint32_t rk_cache_reclaim_for_pages(void *cache, uint32_t pages) { return CACHE->reclaimForPages(pages); }
void rk_cache_poll_transfers(void *cache) { guarded([&] { CACHE->pollTransfers(); return RK_OK; }); }
int rk_cache_compact_extent(void *cache) { return guarded([&] { return CACHE->compactExtent() ? 1 : 0; }); }
int rk_cache_complete_transfer(void *cache, int success) {
  auto *h = static_cast<CacheHandle *>(cache);
  return h->manual && h->manual->complete(success != 0) ? 1 : 0;
}
void rk_cache_manual_tier_set(void *cache, uint32_t transfer_limit, int writable) {
  auto *h = static_cast<CacheHandle *>(cache);
  if (h->manual) h->manual->set(transfer_limit, writable != 0);
}
void rk_cache_manual_tier_plain_limits(void *cache, int plain) {
  auto *h = static_cast<CacheHandle *>(cache);
  if (h->manual) h->manual->setPlainLimits(plain != 0);
}
void rk_cache_tier_counters(const void *cache, uint64_t *out) {
  const auto s = static_cast<const CacheHandle *>(cache)->cache->snapshot();
  out[0] = s.demotionsRefused; out[1] = s.replacedCopies; out[2] = s.cancelledRestores;
  out[3] = s.pendingPages; out[4] = s.demotionsLanded; out[5] = s.restoresLanded;
}
void rk_cache_fail_next_transfers(void *cache, uint32_t count) {
  auto *h = static_cast<CacheHandle *>(cache);
  if (h->host) h->host->failNext(count);
}
void rk_cache_snapshot(const void *cache, uint64_t *out) {
  const auto s = static_cast<const CacheHandle *>(cache)->cache->snapshot();
  out[0] = s.requests; out[1] = s.residentBlocks; out[2] = s.tierBlocks; out[3] = s.transfers; out[4] = s.demotions;
  out[5] = s.restores; out[6] = s.failedTransfers; out[7] = s.evictedBlocks; out[8] = s.forkCopies; out[9] = s.truncatedPages;
}
int rk_cache_block_state(const void *cache, uint64_t block, uint64_t *out) {
  auto &index = static_cast<const CacheHandle *>(cache)->cache->index();
  if (!index.contains(block)) return -1;
  out[0] = index.page(block); out[1] = index.slot(block) != nullptr; out[2] = index.transferring(block); out[3] = index.lastUsed(block);
  out[4] = index.poisoned(block);
  return 0;
}
#undef CACHE

// ---- the slot store: KV that survives a restart (runtime/model/SlotFile.hpp:98-219, records and labels) ----------
void *rk_slot_store_open(const char *slots_path, const char *records_path, const void *tag, uint32_t tag_bytes,
                         uint32_t label_bytes, uint64_t slot_bytes) {
  try {
    model::SlotStore::Persistence persistence;
    persistence.slots = slots_path;
    persistence.records = records_path;
    persistence.tag.assign(static_cast<const uint8_t *>(tag), static_cast<const uint8_t *>(tag) + tag_bytes);
    persistence.labelBytes = label_bytes;
    return new model::SlotStore(slot_bytes, persistence);
  } catch (const std::exception &e) { rk::set_error(e.what()); return nullptr; }
}
void rk_slot_store_close(void *store) { delete static_cast<model::SlotStore *>(store); }
uint32_t rk_slot_store_record_count(const void *store) { return uint32_t(static_cast<const model::SlotStore *>(store)->records().size()); }
int rk_slot_store_record(const void *store, uint32_t at, uint32_t *index, uint64_t *payload_bytes, uint32_t *checksum, void *label) {
  const auto &records = static_cast<const model::SlotStore *>(store)->records();
  if (at >= records.size()) return RK_ERR_INVALID;
  *index = records[at].index;
  *payload_bytes = records[at].payloadBytes;
  *checksum = records[at].checksum;
  if (label) std::memcpy(label, records[at].label.data(), records[at].label.size());
  return RK_OK;
}
int rk_slot_store_write(void *store, uint32_t index, const void *payload, uint64_t payload_bytes, uint32_t checksum, const void *label) {
  auto *s = static_cast<model::SlotStore *>(store);
  return guarded([&] {
    return s->write(index, {static_cast<const uint8_t *>(payload), size_t(payload_bytes)}, checksum,
                    {static_cast<const uint8_t *>(label), s->labelBytes()}) ? RK_OK : RK_ERR_REFUSED;
  });
}
int rk_slot_store_read(const void *store, uint32_t index, void *destination, uint64_t bytes) {
  return guarded([&] { return static_cast<const model::SlotStore *>(store)->read(index, {static_cast<uint8_t *>(destination), size_t(bytes)}) ? RK_OK : RK_ERR_REFUSED; });
}
int rk_slot_store_free(void *store, uint32_t index) { return guarded([&] { return static_cast<model::SlotStore *>(store)->free(index) ? RK_OK : RK_ERR_REFUSED; }); }
int rk_slot_store_synchronize(void *store) { return static_cast<model::SlotStore *>(store)->synchronize() ? RK_OK : RK_ERR_REFUSED; }
uint64_t rk_slot_record_bytes(uint32_t label_bytes) { return model::recordBytesFor(label_bytes); }
// One record / the record file's header as the file holds them (for readers of the format).
int rk_slot_record_encode(uint32_t label_bytes, uint64_t payload_bytes, uint32_t checksum, const void *label, void *out) {
  return guarded([&] {
    const auto record = model::encodeRecord(model::recordBytesFor(label_bytes), payload_bytes, checksum, {static_cast<const uint8_t *>(label), label_bytes});
    std::memcpy(out, record.data(), record.size());
    return RK_OK;
  });
}
int64_t rk_slot_records_header(uint64_t slot_bytes, uint32_t label_bytes, const void *tag, uint32_t tag_bytes, void *out, uint32_t capacity) {
  try {
    const auto header = model::encodeRecordsHeader(slot_bytes, label_bytes, {static_cast<const uint8_t *>(tag), tag_bytes});
    if (header.size() > capacity) return RK_ERR_INVALID;
    std::memcpy(out, header.data(), header.size());
    return int64_t(header.size());
  } catch (const std::exception &e) { rk::set_error(e.what()); return RK_ERR_INVALID; }
}
// Seals the cache's landed tier copies into the store; returns the slots written.
int64_t rk_cache_persist(void *cache, void *store) {
  int64_t written = 0;
  const int status = guarded([&] { written = static_cast<CacheHandle *>(cache)->cache->persist(*static_cast<model::SlotStore *>(store)); return RK_OK; });
  return status ? status : written;
}
// Takes back what an earlier process sealed; out = {blocks, dropped, bytes}.
int rk_cache_adopt(void *cache, void *store, uint64_t *out) {
  return guarded([&] {
    const auto adoption = static_cast<CacheHandle *>(cache)->cache->adopt(*static_cast<model::SlotStore *>(store));
    out[0] = adoption.blocks; out[1] = adoption.dropped; out[2] = adoption.bytes;
    return RK_OK;
  });
}

// The reference's rule for restore points: a stored state comes back with its whole chain, a block only for a state.
// state_labels: `count` StateLabel records of 24 bytes; state_bytes: each state's size. out = {blocks, dropped, bytes, states}.
int rk_cache_adopt_restore_points(void *cache, void *store, const void *state_labels, const uint64_t *state_bytes, uint32_t count, uint64_t *out) {
  return guarded([&] {
    std::vector<engine::Cache::PersistedState> states(count);
    for (uint32_t i = 0; i < count; ++i) {
      std::memcpy(&states[i].label, static_cast<const uint8_t *>(state_labels) + size_t(i) * sizeof(model::StateLabel), sizeof(model::StateLabel));
      states[i].bytes = state_bytes[i];
    }
    const auto adoption = static_cast<CacheHandle *>(cache)->cache->adoptRestorePoints(*static_cast<model::SlotStore *>(store), states);
    out[0] = adoption.blocks; out[1] = adoption.dropped; out[2] = adoption.bytes; out[3] = adoption.states;
    return RK_OK;
  });
}
// The label of every stored state as a clean stop writes it; returns how many there are (the first `capacity` are written).
int64_t rk_cache_state_labels(void *cache, void *labels, uint64_t *state_bytes, uint32_t capacity) {
  int64_t count = -1;
  const int status = guarded([&] {
    const auto found = static_cast<CacheHandle *>(cache)->cache->stateLabels();
    for (size_t i = 0; i < found.size() && i < capacity; ++i) {
      std::memcpy(static_cast<uint8_t *>(labels) + i * sizeof(model::StateLabel), &found[i].label, sizeof(model::StateLabel));
      state_bytes[i] = found[i].bytes;
    }
    count = int64_t(found.size());
    return RK_OK;
  });
  return status == RK_OK ? count : -1;
}

int rk_plan_verify(uint32_t lanes, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t format,
                   const uint32_t *history, int tree, uint32_t row_capacity, uint32_t ctas, char *names, size_t names_bytes, uint64_t *out) {
  return guarded([&] {
    const auto plan = ops::PagedAttention::verifyPlan(lanes, query_heads, layoutOf(layers, kv_heads, head_dim, format), {history, lanes}, tree != 0, row_capacity, ctas);
    if (int s = joinNames({plan.splitPipeline, plan.reducePipeline, plan.storePipeline}, names, names_bytes)) return s;
    size_t i = 0;
    out[i++] = plan.splits;
    for (uint32_t l = 0; l < 4; ++l) out[i++] = l < lanes ? plan.laneSplits[l] : 0;
    out[i++] = plan.splitGroups.x; out[i++] = plan.splitGroups.y; out[i++] = plan.splitGroups.z;
    out[i++] = plan.reduceGroups.x; out[i++] = plan.reduceGroups.y; out[i++] = plan.reduceGroups.z;
    out[i++] = plan.workspace.partialsBytes; out[i++] = plan.workspace.statisticsBytes; out[i++] = plan.rowCapacity;
    out[i++] = plan.streamingDecode; out[i++] = plan.tensorCoreWindow;
    return RK_OK;
  });
}
int rk_plan_window_splits(uint32_t lanes, uint32_t kv_heads, uint32_t visible_tokens, uint32_t ctas) {
  if (!ctas) {
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
      (void)cudaGetLastError();
      rk::set_error("rk_plan_window_splits: no device to size the plan for");
      return RK_ERR_INVALID;
    }
    ctas = uint32_t(sms);
  }
  return int(ops::PagedAttention::windowSplits(lanes, kv_heads, visible_tokens, ctas));
}
int rk_plan_prefill(uint32_t rows, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t format,
                    char *names, size_t names_bytes, uint64_t *out) {
  return guarded([&] {
    const auto plan = ops::PagedAttention::prefillPlan(rows, query_heads, layoutOf(layers, kv_heads, head_dim, format));
    if (int s = joinNames({plan.splitPipeline, plan.reducePipeline}, names, names_bytes)) return s;
    size_t i = 0;
    out[i++] = plan.rows; out[i++] = plan.splits;
    out[i++] = plan.splitGroups.x; out[i++] = plan.splitGroups.y; out[i++] = plan.splitGroups.z;
    out[i++] = plan.reduceGroups.x; out[i++] = plan.reduceGroups.y; out[i++] = plan.reduceGroups.z;
    out[i++] = plan.workspace.partialsBytes; out[i++] = plan.workspace.statisticsBytes;
    return RK_OK;
  });
}
int rk_plan_workspaces(uint32_t lanes, uint32_t max_rows, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim,
                       uint32_t format, uint64_t *out) {
  return guarded([&] {
    const kv::Layout l = layoutOf(layers, kv_heads, head_dim, format);
    const auto v = ops::PagedAttention::verifyWorkspace(lanes, query_heads, l);
    const auto p = ops::PagedAttention::prefillWorkspace(max_rows, query_heads, l);
    out[0] = v.partialsBytes; out[1] = v.statisticsBytes; out[2] = p.partialsBytes; out[3] = p.statisticsBytes;
    return RK_OK;
  });
}
// ---- composite states and the reclaim order they impose --------------------------------------------------------
#define CACHE (static_cast<CacheHandle *>(cache)->cache)
int64_t rk_cache_block_at(void *cache, uint64_t request, uint32_t tokens) {
  int64_t block = 0;
  const int status = guarded([&] { block = int64_t(CACHE->blockAt(request, tokens)); return RK_OK; });
  return status ? status : block;
}
int rk_cache_state_publish(void *cache, uint64_t block, uint64_t bytes, int checkpoint) {
  return guarded([&] { CACHE->publishCompositeState(block, bytes, checkpoint != 0); return RK_OK; });
}
// A state whose only copy the model stores elsewhere (StateCache::publishStateToDisk): no RAM, no reclaim candidate,
// but the KV it restores through stays worth a tier copy.
int rk_cache_state_publish_stored(void *cache, uint64_t block, uint64_t bytes, int checkpoint) {
  return guarded([&] { CACHE->publishStoredState(block, bytes, checkpoint != 0); return RK_OK; });
}
int rk_cache_state_use(void *cache, uint64_t block, int use) {
  return guarded([&] { if (use) CACHE->states().use(block); else CACHE->states().unuse(block); return RK_OK; });
}
int rk_cache_state_pin(void *cache, uint64_t block, int pin) {
  return guarded([&] { if (pin) CACHE->states().pin(block); else CACHE->states().unpin(block); return RK_OK; });
}
// out[7] = contains, ordinary, in use, bytes, KV needed by a state, KV needed by a state in use, has a RAM copy
int rk_cache_state_info(void *cache, uint64_t block, uint64_t *out) {
  return guarded([&] {
    const engine::StateCache &states = CACHE->states();
    out[0] = states.contains(block); out[1] = states.ordinary(block); out[2] = states.inUse(block); out[3] = states.bytes(block);
    out[4] = CACHE->index().contains(block) && CACHE->kvNeededByState(block);
    out[5] = CACHE->index().contains(block) && CACHE->kvNeededByStateInUse(block);
    out[6] = states.stateResident(block);
    return RK_OK;
  });
}
// out[4] = states, resident bytes, evictable states (with those in use), resume point
int rk_cache_state_summary(void *cache, uint64_t *out) {
  return guarded([&] {
    const engine::StateCache &states = CACHE->states();
    out[0] = states.size(); out[1] = states.residentBytes(); out[2] = states.evictableStates(true); out[3] = states.resumePoint();
    return RK_OK;
  });
}
// One eviction step in the reference's order; out[4] = made progress, pending, evicted a state, state bytes freed.
int rk_cache_evict_one(void *cache, int up_to_in_use, int keep_resume_point, int pages_only, uint64_t *out) {
  return guarded([&] {
    const engine::ReclaimStep step = CACHE->evictOne(up_to_in_use ? engine::ReclaimClass::InUse : engine::ReclaimClass::Ordinary,
                                                     keep_resume_point != 0, pages_only != 0);
    out[0] = step.madeProgress; out[1] = step.pending; out[2] = step.evictedState; out[3] = step.reclaimedBytes;
    return RK_OK;
  });
}
// Cache::reclaimOne(mode, upTo, keepResumePoint, keepRunway): mode 0 = release extents, 1 = keep extents, 2 = reuse
// pages. out[4] as rk_cache_evict_one, reclaimed bytes counting returned extents too.
int rk_cache_reclaim_step(void *cache, int mode, int up_to_in_use, int keep_resume_point, int keep_runway, uint64_t *out) {
  return guarded([&] {
    if (mode < 0 || mode > 2) throw std::invalid_argument("unknown reclaim mode");
    const engine::ReclaimStep step = CACHE->reclaimStep(engine::Cache::ReclaimMode(mode), up_to_in_use ? engine::ReclaimClass::InUse : engine::ReclaimClass::Ordinary,
                                                        keep_resume_point != 0, keep_runway != 0);
    out[0] = step.madeProgress; out[1] = step.pending; out[2] = step.evictedState; out[3] = step.reclaimedBytes;
    return RK_OK;
  });
}
// Cache::evictAll: out[2] = made progress, extent bytes returned
int rk_cache_evict_all(void *cache, uint64_t *out) {
  return guarded([&] {
    const engine::ReclaimStep step = CACHE->evictAll();
    out[0] = step.madeProgress; out[1] = step.reclaimedBytes;
    return RK_OK;
  });
}
int rk_cache_reclaim_one_state(void *cache, int checkpoints_only, uint64_t for_block) {
  return guarded([&] { return CACHE->reclaimOneState(checkpoints_only != 0, for_block) ? 1 : 0; });
}
// Cache::lookup of a hybrid model's admission: the chain into blocks_out (returns its length), out[5] = KV boundary,
// state block (pinned for the caller; 0 = none), resume boundary, junction boundary, lost state. `record` counts the
// lookup as Cache::recordLookup does. `probe` (may be null) is a handle of rk_cache_probe_create: while it is current
// its chain is reused instead of hashing the prompt again.
int64_t rk_cache_lookup_state(void *cache, const uint32_t *prompt, uint32_t prompt_tokens, uint64_t *blocks_out, uint32_t capacity,
                              uint64_t *out, int record, const void *probe, const rk_image_span *images, uint32_t image_count) {
  try {
    const auto found = CACHE->lookupWithState({prompt, prompt_tokens}, static_cast<const engine::Cache::Probe *>(probe),
                                              image_spans(images, image_count));
    for (size_t i = 0; i < found.blocks.size() && i < capacity; ++i) blocks_out[i] = found.blocks[i];
    out[0] = found.kvBoundary; out[1] = found.stateBlock; out[2] = found.resumeBoundary; out[3] = found.junctionBoundary;
    out[4] = found.lostState;
    if (record) CACHE->recordLookup(found);
    return int64_t(found.blocks.size());
  } catch (const std::exception &e) { rk::set_error(e.what()); return RK_ERR_INVALID; }
}
// out[4] = KV tokens hit, lookups at a branch point with a state below (lazy junctions), lookups that met a lost
// state, pages hashed by scheduling probes
int rk_cache_lookup_counters(void *cache, uint64_t *out) {
  return guarded([&] {
    const auto counters = CACHE->lookupCounters();
    out[0] = counters.kvHitTokens; out[1] = counters.lazyJunctions; out[2] = counters.lostStateMisses;
    out[3] = counters.probeHashedBlocks;
    return RK_OK;
  });
}
// The scheduling probe (Cache::probe / Cache::refresh / CacheProbe): a handle the scheduler keeps per waiting request.
void *rk_cache_probe_create(void *cache, const uint32_t *prompt, uint32_t prompt_tokens, const rk_image_span *images, uint32_t image_count) {
  try { return new engine::Cache::Probe(CACHE->probe({prompt, prompt_tokens}, image_spans(images, image_count))); }
  catch (const std::exception &e) { rk::set_error(e.what()); return nullptr; }
}
int rk_cache_probe_refresh(void *cache, void *probe, const uint32_t *prompt, uint32_t prompt_tokens, const rk_image_span *images,
                           uint32_t image_count) {
  return guarded([&] {
    CACHE->refresh(*static_cast<engine::Cache::Probe *>(probe), {prompt, prompt_tokens}, image_spans(images, image_count));
    return RK_OK;
  });
}
// out[2] = cached tokens (up to the deepest state on the matched chain), matched blocks
int rk_cache_probe_info(const void *probe, uint64_t *out) {
  return guarded([&] {
    const auto *held = static_cast<const engine::Cache::Probe *>(probe);
    out[0] = held->cachedTokens(); out[1] = held->blocks().size();
    return RK_OK;
  });
}
void rk_cache_probe_destroy(void *probe) { delete static_cast<engine::Cache::Probe *>(probe); }

#undef CACHE

// ---- the operator's encoders (ops::PagedAttention::add*): validation first, then the launches ------------------
namespace {
struct OperatorPlan {
  bool verify = false;
  kv::Layout layout{};
  uint32_t queryHeads = 0;
  ops::VerifyAttentionPlan verifyPlan{};
  ops::PrefillAttentionPlan prefillPlan{};
};
} // namespace

void *rk_op_verify_plan(uint32_t lanes, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t format,
                        const uint32_t *history, int tree, uint32_t row_capacity, uint32_t ctas) {
  OperatorPlan *plan = nullptr;
  guarded([&] {
    auto made = std::make_unique<OperatorPlan>();
    made->verify = true;
    made->layout = layoutOf(layers, kv_heads, head_dim, format);
    made->queryHeads = query_heads;
    made->verifyPlan = ops::PagedAttention::verifyPlan(lanes, query_heads, made->layout, {history, lanes}, tree != 0, row_capacity, ctas);
    plan = made.release();
    return RK_OK;
  });
  return plan;
}
void *rk_op_prefill_plan(uint32_t rows, uint32_t query_heads, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t format) {
  OperatorPlan *plan = nullptr;
  guarded([&] {
    auto made = std::make_unique<OperatorPlan>();
    made->layout = layoutOf(layers, kv_heads, head_dim, format);
    made->queryHeads = query_heads;
    made->prefillPlan = ops::PagedAttention::prefillPlan(rows, query_heads, made->layout);
    plan = made.release();
    return RK_OK;
  });
  return plan;
}
void rk_op_plan_destroy(void *plan) { delete static_cast<OperatorPlan *>(plan); }
int rk_op_plan_workspace(const void *plan, uint64_t *out) {
  const auto *p = static_cast<const OperatorPlan *>(plan);
  if (!p || !out) { rk::set_error("rk_op_plan_workspace: invalid arguments"); return RK_ERR_INVALID; }
  const ops::AttentionWorkspace &w = p->verify ? p->verifyPlan.workspace : p->prefillPlan.workspace;
  out[0] = w.partialsBytes; out[1] = w.statisticsBytes;
  out[2] = p->verify ? p->verifyPlan.splits : p->prefillPlan.splits;
  out[3] = p->verify ? p->verifyPlan.rowCapacity : p->prefillPlan.rows;
  out[4] = p->verify ? uint64_t(p->verifyPlan.streamingDecode) | (uint64_t(p->verifyPlan.tensorCoreWindow) << 1) : 0;
  out[5] = p->verify ? p->verifyPlan.decode.descriptor_bytes : 0;
  return RK_OK;
}
uint32_t rk_op_plan_lane_splits(const void *plan, uint32_t lane) {
  const auto *p = static_cast<const OperatorPlan *>(plan);
  return p && p->verify && lane < p->verifyPlan.laneSplits.size() ? p->verifyPlan.laneSplits[lane] : 0;
}

int rk_op_add_prefill_store(void *stream, rk_kv_layer layer, const void *chunk_keys, const void *chunk_values, const rk_page_entry *table,
                            const rk_chunk_params *params, uint32_t layers, uint32_t kv_heads, uint32_t head_dim, uint32_t format) {
  return guarded([&] {
    if (!params) throw std::invalid_argument("invalid paged prefill store");
    ops::PagedAttention::addPrefillStore(stream, layer, chunk_keys, chunk_values, table, *params, layoutOf(layers, kv_heads, head_dim, format));
    return RK_OK;
  });
}
int rk_op_add_prefill(void *stream, rk_kv_layer layer, const void *queries, void *output, float *partials, float *statistics,
                      uint64_t partials_bytes, uint64_t statistics_bytes, const rk_page_entry *table, const rk_chunk_params *chunk,
                      const void *plan, const void *window, uint32_t *status) {
  return guarded([&] {
    const auto *p = static_cast<const OperatorPlan *>(plan);
    if (!p || p->verify || !chunk) throw std::invalid_argument("prefill attention needs a prefill plan");
    ops::PagedAttention::addPrefill(stream, layer, queries, output, partials, statistics, partials_bytes, statistics_bytes, table, *chunk,
                                    p->prefillPlan, p->queryHeads, p->layout, window, status);
    return RK_OK;
  });
}
int rk_op_add_verify(void *stream, rk_kv_layer layer, const rk_verify_buffers *buffers, const rk_chunk_params *device_chunks,
                     const rk_verify_params *device_attention, const void *plan, const void *window) {
  return guarded([&] {
    const auto *p = static_cast<const OperatorPlan *>(plan);
    if (!p || !p->verify || !buffers) throw std::invalid_argument("verify attention needs a verify plan");
    ops::PagedVerifyBuffers b;
    b.chunkKeys = buffers->chunk_keys; b.chunkValues = buffers->chunk_values; b.queries = buffers->queries; b.output = buffers->output;
    b.partials = buffers->partials; b.statistics = buffers->statistics; b.descriptors = buffers->descriptors; b.status = buffers->status;
    b.pageTables = buffers->page_tables; b.treeMasks = buffers->tree_masks;
    b.partialsBytes = buffers->partials_bytes; b.statisticsBytes = buffers->statistics_bytes;
    ops::PagedAttention::addVerify(stream, layer, b, device_chunks, device_attention, p->verifyPlan, p->queryHeads, p->layout, window);
    return RK_OK;
  });
}
int rk_op_add_verify_tree_compact(void *stream, rk_kv_layer layer, const rk_page_entry *const *page_tables, const uint32_t *retained_path,
                                  const uint32_t *retained, const rk_chunk_params *device_chunks, uint32_t lanes, uint32_t layers,
                                  uint32_t kv_heads, uint32_t head_dim, uint32_t format) {
  return guarded([&] {
    ops::PagedAttention::addVerifyTreeCompact(stream, layer, page_tables, retained_path, retained, device_chunks, lanes,
                                              layoutOf(layers, kv_heads, head_dim, format));
    return RK_OK;
  });
}

const char *rk_chunk_validation_error(uint32_t committed, uint32_t tokens, uint32_t stride, uint32_t entries) {
  static thread_local std::string text;
  text = std::string(ops::chunkedPrefillValidationError(rk_chunk_params{committed, tokens, stride, entries, {0, 0}}));
  return text.c_str();
}

} // extern "C"
