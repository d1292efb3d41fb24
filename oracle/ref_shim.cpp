// ref_shim.cpp — C entry points over the reference's OWN portable code, compiled
// in place from the reference checkout (never copied into this repository).
//
// TEST INFRASTRUCTURE ONLY. Built by oracle/Makefile into oracle/_ref/ when the
// reference checkout is present; used to pin the C++ restatement (rk_oracle.cpp)
// and the host control plane against the reference itself:
//   dev/tests/engine/Q8PageFormatReference.hpp   int8 page quantizer, bf16 conversion
//   dev/tests/engine/Fp8PageFormatReference.hpp  e4m3 encode/decode, fp16 query staging
//   runtime/ops/PagedKv.hpp                      kv::Layout byte and extent accounting
//   runtime/metal/abi/KvExtent.h                 offsets and page entries
//   runtime/ops/PagedAttention.{hpp,cpp}         plans: kernel names, grids, workspaces
//   runtime/engine/cache/KvPool.{hpp,cpp}        the page allocator
//   runtime/model/SlotFile.{hpp,cpp}, Crc32c.hpp   the persistent slot file and its record file (Darwin's fcntl
//                                                commands and the ARM CRC intrinsics stood in for by
//                                                darwin_clock_shim.h and darwin_shim/arm_acle.h)
//   runtime/engine/cache/{Cache,KvCache,StateCache}.{hpp,cpp}  the request cache facade, its block graph and the
//                                                state cache it couples KV reclaim to, over the reference's own test
//                                                tier (dev/tests/engine/TestKvTier.hpp)
#include "Q8PageFormatReference.hpp"
#include "Fp8PageFormatReference.hpp"
#include "engine/cache/Cache.hpp"
#include "engine/cache/DiskLabels.hpp"
#include "engine/cache/KvPool.hpp"
#include "model/SlotFile.hpp"
#include "TestKvTier.hpp"
#include "ops/PagedAttention.hpp"

#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <vector>

using namespace richengine;

// PagedAttention.cpp references two helpers of the linear operator that the
// plan and store/attention encoders never reach with a Plain input; the
// checker does not build the linear operator, so they are defined here to
// refuse loudly.
namespace richengine::ops {
void requireTableScratch(const LinearScratch &, LinearInput, uint32_t, uint32_t) {
  throw std::logic_error("linear table scratch is outside the checker");
}
const char *tableSuffix(LinearInput) noexcept { return ""; }
} // namespace richengine::ops


// The plan encoders name the backend's buffer handle; the checker has no Metal
// backend, so the handle is an empty reference that is never bound.
namespace richengine::metal {
struct MetalBuffer::Impl {};
MetalBuffer::MetalBuffer() = default;
MetalBuffer::~MetalBuffer() = default;
MetalBuffer::MetalBuffer(const MetalBuffer &) = default;
MetalBuffer &MetalBuffer::operator=(const MetalBuffer &) = default;
MetalBuffer::MetalBuffer(MetalBuffer &&) noexcept = default;
MetalBuffer &MetalBuffer::operator=(MetalBuffer &&) noexcept = default;
MetalBuffer::operator bool() const noexcept { return false; }
uint64_t MetalBuffer::sizeBytes() const noexcept { return 0; }
} // namespace richengine::metal

namespace {

kv::Layout layout_of(uint32_t layers, uint32_t heads, uint32_t dim, uint32_t format, float scale) {
  return kv::Layout{layers, heads, dim, static_cast<kv::Format>(format), scale};
}

// ExtentStorage without memory: a page budget decides whether growth is granted.
class BudgetStorage final : public kv::ExtentStorage {
public:
  BudgetStorage(uint32_t pages, uint64_t bytes, uint32_t extent)
      : pages_(pages), bytes_(bytes), extent_(extent), allocated_(pages / extent) {}
  uint32_t pageCount() const noexcept override { return pages_; }
  uint64_t bytesPerPage() const noexcept override { return bytes_; }
  uint32_t extentPages() const noexcept override { return extent_; }
  metal::AllocationResult allocateExtent(uint32_t extent) override {
    if (allocated_.at(extent)) throw std::logic_error("extent already allocated");
    uint32_t held = 0;
    for (bool a : allocated_) held += a;
    if (uint64_t(held + 1) * extent_ > budget) return metal::AllocationFailure::EngineBudget;
    allocated_[extent] = true;
    return {};
  }
  void releaseExtent(uint32_t extent) override {
    if (!allocated_.at(extent)) throw std::logic_error("extent not allocated");
    allocated_[extent] = false;
  }
  void copyPages(std::span<const kv::PageCopy> copies) override {
    for (const kv::PageCopy &c : copies) log.push_back(c);
  }
  uint64_t budget = ~0ull;
  std::vector<kv::PageCopy> log;

private:
  uint32_t pages_;
  uint64_t bytes_;
  uint32_t extent_;
  std::vector<bool> allocated_;
};

// A composite state that is a byte count in RAM, nothing else (the reference's own tests use the same, TestState).
class ByteState final : public CompositeState {
public:
  explicit ByteState(uint64_t bytes) : bytes_(bytes) {}
  uint64_t bytes() const noexcept override { return bytes_; }
private:
  uint64_t bytes_;
};

// A state whose only copy is stored elsewhere (and, below, the ticket of a write that has landed already): a byte count, and the label a persistent cache keeps with it (CompositeState::label). The
// copies alive are listed so that a test can read the labels as the next process would find them.
class StoredState final : public CompositeState {
public:
  explicit StoredState(uint64_t bytes) : bytes_(bytes) { alive().insert(this); }
  ~StoredState() override { alive().erase(this); }
  uint64_t bytes() const noexcept override { return bytes_; }
  uint64_t residentBytes() const noexcept override { return 0; }
  void label(std::vector<std::byte> bytes) const override { label_ = std::move(bytes); }
  const std::vector<std::byte> &kept() const noexcept { return label_; }
  static std::set<const StoredState *> &alive() { static std::set<const StoredState *> copies; return copies; }
private:
  uint64_t bytes_;
  mutable std::vector<std::byte> label_;
};
struct LandedWrite final : StateOffload {
  std::shared_ptr<const CompositeState> copy;
  bool ready() const noexcept override { return true; }
  bool finish() override { return true; }
  const std::shared_ptr<const CompositeState> &state() const noexcept override { return copy; }
};

// The reference's facade over the budgeted storage and its test tier.
struct Facade {
  BudgetStorage storage;
  engine::KvPool pool;
  std::unique_ptr<test::TestKvTier> tier;
  engine::Cache cache;
  std::map<uint64_t, engine::StateUse> uses;      // one use handle per block
  std::map<uint64_t, engine::CacheLookup> held;   // lookups kept alive: their leases pin the state
  uint64_t nextHeld = 1;
  Facade(uint32_t pages, uint64_t bytes, uint32_t extent, uint32_t runway, uint64_t budget, int withTier)
      : storage(pages, bytes, extent), pool((storage.budget = budget, storage), runway),
        tier(withTier ? std::make_unique<test::TestKvTier>(withTier == 2) : nullptr), cache(pool, tier.get(), nullptr) {}
};

struct Pool {
  BudgetStorage storage;
  std::unique_ptr<engine::KvPool> pool;
  Pool(uint32_t pages, uint64_t bytes, uint32_t extent) : storage(pages, bytes, extent) {}
};

} // namespace

extern "C" {

uint16_t ref_f32_to_bf16(float v) { return kv::floatToBFloat16(v); }
float ref_bf16_to_f32(uint16_t b) { return kv::bfloat16ToFloat(b); }
uint8_t ref_f32_to_e4m3(float v) { return kv::floatToFp8E4m3(v); }
float ref_e4m3_to_f32(uint8_t c) { return kv::fp8E4m3ToFloat(c); }
float ref_query_stage(float v) { return kv::queryStage(v); }

// Logical [token][head][dim] fp32 rows -> one reference layer page
// (K data, K scales, V data, V scales contiguous: 66 560 bytes at 4 x 256).
int ref_q8_quantize_page(const float *keys, const float *values, uint32_t valid_tokens, void *out) {
  try {
    auto page = std::make_unique<kv::Q8LayerPage>();
    const size_t n = size_t(valid_tokens) * kv::kKvHeads * kv::kHeadDimension;
    kv::quantizeLayerPage({keys, n}, {values, n}, valid_tokens, *page);
    std::memcpy(out, page.get(), sizeof(kv::Q8LayerPage));
    return 0;
  } catch (...) { return -1; }
}

int ref_fp8_quantize_page(const float *keys, const float *values, uint32_t valid_tokens, void *out) {
  try {
    auto page = std::make_unique<kv::Fp8LayerPage>();
    const size_t n = size_t(valid_tokens) * kv::kFp8KvHeads * kv::kFp8HeadDimension;
    kv::quantizeFp8LayerPage({keys, n}, {values, n}, valid_tokens, *page);
    std::memcpy(out, page.get(), sizeof(kv::Fp8LayerPage));
    return 0;
  } catch (...) { return -1; }
}

// out[0..7] = dataBytesPerLayerPage, scaleBytesPerLayerPage, bytesPerLayerPage,
// bytesPerModelPage, extentAlignmentPages, minimumExtentPages, maximumExtentPages,
// extentPagesFor(pool_pages)
void ref_layout(uint32_t layers, uint32_t heads, uint32_t dim, uint32_t format, uint64_t pool_pages,
                uint64_t *out) {
  const kv::Layout l = layout_of(layers, heads, dim, format, 0.0f);
  out[0] = l.dataBytesPerLayerPage();
  out[1] = l.scaleBytesPerLayerPage();
  out[2] = l.bytesPerLayerPage();
  out[3] = l.bytesPerModelPage();
  out[4] = l.extentAlignmentPages();
  out[5] = l.minimumExtentPages();
  out[6] = l.maximumExtentPages();
  out[7] = l.extentPagesFor(pool_pages);
}

uint64_t ref_kv_offset(uint32_t extent_pages, uint32_t data, uint32_t scale, uint32_t layer,
                       uint32_t tensor, uint32_t index) {
  return richengine_kv_offset(extent_pages, data, scale, layer, tensor, index);
}
uint64_t ref_key_element(uint32_t h, uint32_t t, uint32_t d, uint32_t dim) {
  return richengine_kv_key_element_dim(h, t, d, dim);
}
uint64_t ref_value_element(uint32_t h, uint32_t t, uint32_t d, uint32_t dim) {
  return richengine_kv_value_element_dim(h, t, d, dim);
}
uint64_t ref_scale_element(uint32_t h, uint32_t t) { return richengine_kv_scale_element(h, t); }
uint32_t ref_verify_splits(uint32_t committed, uint32_t rows) {
  return kv::verifyAttentionSplits(committed, rows);
}
// Empty string when the chunk is valid, else the reference's error tag.
const char *ref_chunk_validation(uint32_t committed, uint32_t tokens, uint32_t stride, uint32_t entries) {
  static thread_local std::string text;
  kv::ChunkedPrefillParams p{committed, tokens, stride, entries, {}};
  text = std::string(kv::chunkedPrefillValidationError(p));
  return text.c_str();
}

// Verify plan: names joined by '\n' into `names` (split, reduce), numbers into out:
// [splits, lane_splits[4], splitGroups xyz, reduceGroups xyz, partialsBytes,
//  statisticsBytes, rowCapacity]. Returns 0 or -1 when the reference throws.
int ref_verify_plan(uint32_t lanes, uint32_t query_heads, uint32_t layers, uint32_t heads, uint32_t dim,
                    uint32_t format, const uint32_t *history, int tree, char *names, size_t names_bytes,
                    uint64_t *out) {
  try {
    const auto plan = ops::PagedAttention::verifyPlan(
        lanes, query_heads, layout_of(layers, heads, dim, format, 0.0f), {history, lanes}, tree != 0);
    const std::string joined = plan.splitPipeline + "\n" + plan.reducePipeline;
    if (joined.size() + 1 > names_bytes) return -1;
    std::memcpy(names, joined.c_str(), joined.size() + 1);
    size_t i = 0;
    out[i++] = plan.splits;
    for (uint32_t l = 0; l < 4; ++l) out[i++] = plan.laneSplits[l];
    out[i++] = plan.splitGroups.x; out[i++] = plan.splitGroups.y; out[i++] = plan.splitGroups.z;
    out[i++] = plan.reduceGroups.x; out[i++] = plan.reduceGroups.y; out[i++] = plan.reduceGroups.z;
    out[i++] = plan.workspace.partialsBytes;
    out[i++] = plan.workspace.statisticsBytes;
    out[i++] = plan.rowCapacity;
    return 0;
  } catch (...) { return -1; }
}

// Prefill plan: out = [rows, splits, splitGroups xyz, reduceGroups xyz,
// partialsBytes, statisticsBytes].
int ref_prefill_plan(uint32_t rows, uint32_t query_heads, uint32_t layers, uint32_t heads, uint32_t dim,
                     uint32_t format, char *names, size_t names_bytes, uint64_t *out) {
  try {
    const auto plan = ops::PagedAttention::prefillPlan(rows, query_heads,
                                                       layout_of(layers, heads, dim, format, 0.0f));
    const std::string joined = plan.splitPipeline + "\n" + plan.reducePipeline;
    if (joined.size() + 1 > names_bytes) return -1;
    std::memcpy(names, joined.c_str(), joined.size() + 1);
    size_t i = 0;
    out[i++] = plan.rows; out[i++] = plan.splits;
    out[i++] = plan.splitGroups.x; out[i++] = plan.splitGroups.y; out[i++] = plan.splitGroups.z;
    out[i++] = plan.reduceGroups.x; out[i++] = plan.reduceGroups.y; out[i++] = plan.reduceGroups.z;
    out[i++] = plan.workspace.partialsBytes;
    out[i++] = plan.workspace.statisticsBytes;
    return 0;
  } catch (...) { return -1; }
}

int ref_workspaces(uint32_t lanes, uint32_t max_rows, uint32_t query_heads, uint32_t layers,
                   uint32_t heads, uint32_t dim, uint32_t format, uint64_t *out) {
  try {
    const kv::Layout l = layout_of(layers, heads, dim, format, 0.0f);
    const auto v = ops::PagedAttention::verifyWorkspace(lanes, query_heads, l);
    const auto p = ops::PagedAttention::prefillWorkspace(max_rows, query_heads, l);
    out[0] = v.partialsBytes; out[1] = v.statisticsBytes;
    out[2] = p.partialsBytes; out[3] = p.statisticsBytes;
    return 0;
  } catch (...) { return -1; }
}

// ---- the reference allocator over a budgeted fake storage --------------------
void *ref_pool_create(uint32_t pages, uint64_t bytes_per_page, uint32_t extent_pages,
                      uint32_t runway_pages, uint64_t budget_pages) {
  try {
    auto holder = std::make_unique<Pool>(pages, bytes_per_page, extent_pages);
    holder->storage.budget = budget_pages;
    holder->pool = std::make_unique<engine::KvPool>(holder->storage, runway_pages);
    return holder.release();
  } catch (...) { return nullptr; }
}
void ref_pool_destroy(void *pool) { delete static_cast<Pool *>(pool); }
void ref_pool_set_budget(void *pool, uint64_t budget_pages) {
  static_cast<Pool *>(pool)->storage.budget = budget_pages;
}
// Returns the number granted (count) or -1 when refused; pages into out.
int ref_pool_acquire(void *pool, uint32_t count, uint32_t *out) {
  try {
    auto got = static_cast<Pool *>(pool)->pool->acquirePages(count);
    if (!got.granted()) return -1;
    std::copy(got.pages.begin(), got.pages.end(), out);
    return int(got.pages.size());
  } catch (...) { return -2; }
}
int ref_pool_retain(void *pool, uint32_t page, int prefix) {
  try { static_cast<Pool *>(pool)->pool->retainPage(page, prefix != 0); return 0; } catch (...) { return -1; }
}
int ref_pool_release(void *pool, uint32_t page, int prefix) {
  try { static_cast<Pool *>(pool)->pool->releasePage(page, prefix != 0); return 0; } catch (...) { return -1; }
}
uint64_t ref_pool_reclaim(void *pool, int keep_runway, uint32_t limit) {
  return static_cast<Pool *>(pool)->pool->reclaimEmptyExtents(keep_runway != 0, limit);
}
// Moves: destinations (extent_pages entries) into out; returns first page or -1 when nothing moved.
int64_t ref_pool_compact(void *pool, const uint32_t *fixed, uint32_t fixed_count, uint32_t *out) {
  auto moves = static_cast<Pool *>(pool)->pool->compactExtent({fixed, fixed_count});
  if (moves.empty()) return -1;
  std::copy(moves.destinations.begin(), moves.destinations.end(), out);
  return moves.firstPage;
}
// out = [pagesAllocated, pagesFree, pagesActive, pagesPrefix, allocatedBytes,
//        reclaimableBytes, extentAllocations, extentReleases, extentCompactions, pagesMoved]
void ref_pool_snapshot(void *pool, uint64_t *out) {
  const auto s = static_cast<Pool *>(pool)->pool->snapshot();
  out[0] = s.pagesAllocated; out[1] = s.pagesFree; out[2] = s.pagesActive; out[3] = s.pagesPrefix;
  out[4] = s.allocatedBytes; out[5] = s.reclaimableBytes; out[6] = s.extentAllocations;
  out[7] = s.extentReleases; out[8] = s.extentCompactions; out[9] = s.pagesMoved;
}


// ---- the reference's request cache facade -------------------------------------------------
#define FACADE (static_cast<Facade *>(facade))
void *ref_cache_create(uint32_t pages, uint64_t bytes_per_page, uint32_t extent_pages, uint32_t runway_pages,
                       uint64_t budget_pages, int with_tier, uint32_t tier_capacity, uint32_t transfer_limit) {
  try {
    auto f = std::make_unique<Facade>(pages, bytes_per_page, extent_pages, runway_pages, budget_pages, with_tier); // 2: a persistent tier
    if (f->tier) { f->tier->capacity = tier_capacity; f->tier->transferLimit = transfer_limit; }
    return f.release();
  } catch (...) { return nullptr; }
}
void ref_cache_destroy(void *facade) {
  if (!facade) return;
  FACADE->held.clear();
  FACADE->uses.clear();
  if (FACADE->tier) FACADE->tier->complete();
  delete FACADE;
}
void ref_cache_tier_set(void *facade, uint32_t transfer_limit, int writable) {
  if (!FACADE->tier) return;
  FACADE->tier->transferLimit = transfer_limit;
  FACADE->tier->writableFile = writable != 0;
}
void ref_cache_tier_complete(void *facade, int success) { if (FACADE->tier) FACADE->tier->complete(success != 0); }
int ref_cache_begin(void *facade, uint64_t request) { try { FACADE->cache.beginRequest(request); return 0; } catch (...) { return -1; } }
int ref_cache_end(void *facade, uint64_t request) { try { FACADE->cache.endRequest(request); return 0; } catch (...) { return -1; } }
// 0 granted, 1 denied, 2 pending, -1 threw
int ref_cache_ensure(void *facade, uint64_t request, uint64_t tokens) {
  try { return int(FACADE->cache.ensureTokens(request, tokens).failure); } catch (...) { return -1; }
}
int64_t ref_cache_page_table(void *facade, uint64_t request, uint32_t *pages, uint32_t capacity, uint64_t *revision, uint32_t *first_changed) {
  try {
    const auto view = FACADE->cache.pageTable(request);
    for (size_t i = 0; i < view.pages.size() && i < capacity; ++i) pages[i] = view.pages[i];
    *revision = view.revision; *first_changed = view.firstChanged;
    return int64_t(view.pages.size());
  } catch (...) { return -1; }
}
// Image spans cross as the 32-byte records of include/richkv_host.h, which are ImageSpan's own fields in its order.
static std::span<const ImageSpan> spans_of(const void *images, uint32_t count) {
  static_assert(sizeof(ImageSpan) == 32);
  return {static_cast<const ImageSpan *>(images), images ? count : 0u};
}
int ref_cache_publish(void *facade, uint64_t request, const uint32_t *tokens, uint32_t count, uint32_t committed, const void *images, uint32_t image_count) {
  try { FACADE->cache.publishCommittedBlocks(request, {tokens, count}, committed, spans_of(images, image_count)); return 0; } catch (...) { return -1; }
}
// blockImageIdentity (runtime/engine/cache/KvCache.cpp:29-52): out[2] = lo, hi
void ref_block_image_identity(uint64_t block_begin, uint32_t block_tokens, const void *images, uint32_t image_count, uint64_t *out) {
  const engine::ImageIdentity identity = engine::blockImageIdentity(block_begin, block_tokens, spans_of(images, image_count));
  out[0] = identity.lo; out[1] = identity.hi;
}
uint64_t ref_cache_block_at(void *facade, uint64_t request, uint32_t boundary) {
  try { return FACADE->cache.blockAt(request, boundary); } catch (...) { return 0; }
}
// out[5] = kv boundary, state block, resume boundary, junction boundary, lost state. hold != 0 keeps the lookup (its
// lease pins the state) and returns its handle in out[5]; attach_to != 0 gives that request the chain (restoreRequest)
// and reports the admission in out[6] (0 granted, 1 denied, 2 pending).
int ref_cache_lookup(void *facade, const uint32_t *prompt, uint32_t count, int record, int hold, uint64_t attach_to, uint64_t *out,
                     const void *probe, const void *images, uint32_t image_count) {
  try {
    engine::CacheLookup found = FACADE->cache.lookup({prompt, count}, spans_of(images, image_count), static_cast<const engine::CacheProbe *>(probe));
    out[0] = found.kvBoundary; out[1] = found.state ? found.state->kvBlock() : 0; out[2] = found.resumeBoundary();
    out[3] = found.junctionBoundary; out[4] = found.lostState; out[5] = 0; out[6] = 0;
    if (record) FACADE->cache.recordLookup(found);
    if (attach_to) out[6] = uint64_t(FACADE->cache.restoreRequest(attach_to, found).failure);
    if (hold) { out[5] = FACADE->nextHeld; FACADE->held.emplace(FACADE->nextHeld++, std::move(found)); }
    return 0;
  } catch (...) { return -1; }
}
void ref_cache_release_lookup(void *facade, uint64_t handle) { FACADE->held.erase(handle); }
void *ref_cache_probe_create(void *facade, const uint32_t *prompt, uint32_t count, const void *images, uint32_t image_count) {
  try { return new engine::CacheProbe(FACADE->cache.probe({prompt, count}, spans_of(images, image_count))); } catch (...) { return nullptr; }
}
int ref_cache_probe_refresh(void *facade, void *probe, const uint32_t *prompt, uint32_t count, const void *images, uint32_t image_count) {
  try { FACADE->cache.refresh(*static_cast<engine::CacheProbe *>(probe), {prompt, count}, spans_of(images, image_count)); return 0; } catch (...) { return -1; }
}
uint32_t ref_cache_probe_cached_tokens(const void *probe) { return static_cast<const engine::CacheProbe *>(probe)->cachedTokens(); }
void ref_cache_probe_destroy(void *probe) { delete static_cast<engine::CacheProbe *>(probe); }
int ref_cache_restore_status(void *facade, uint64_t request) {
  try { return int(FACADE->cache.kvRestoreStatus(request)); } catch (...) { return -1; }
}
int ref_cache_publish_state(void *facade, uint64_t block, uint64_t bytes, int checkpoint) {
  try { // as the engine does: the state that is there is reused, a publication follows only without one
    if (!FACADE->cache.reuseCompositeState(block, checkpoint != 0))
      FACADE->cache.publishCompositeState(block, std::make_shared<ByteState>(bytes), checkpoint != 0);
    return 0;
  } catch (...) { return -1; }
}
// StateCache::publishStateToDisk with a write that lands at once; the poll that follows retires it.
int ref_cache_publish_state_stored(void *facade, uint64_t block, uint64_t bytes, int checkpoint) {
  try {
    const bool taken = FACADE->cache.publishStateToDisk(block, [bytes](std::function<void()>) {
      auto ticket = std::make_unique<LandedWrite>();
      ticket->copy = std::make_shared<StoredState>(bytes);
      return std::unique_ptr<StateOffload>(std::move(ticket));
    }, checkpoint != 0);
    return taken ? 0 : 1;
  } catch (...) { return -1; }
}
int ref_cache_use_state(void *facade, uint64_t block, int use) {
  try {
    if (use) FACADE->uses[block] = FACADE->cache.useState(block);
    else FACADE->uses.erase(block);
    return 0;
  } catch (...) { return -1; }
}
// out[4] = made progress, pending, evicted a state, reclaimed bytes
int ref_cache_evict_one(void *facade, int up_to_in_use, int keep_resume_point, int pages_only, uint64_t *out) {
  try {
    // evictOne is private: reclaimOne(KeepExtents | ReusePages) is evictOne(upTo, keepResumePoint, pagesOnly)
    const auto step = FACADE->cache.reclaimOne(pages_only ? engine::CacheReclaimMode::ReusePages : engine::CacheReclaimMode::KeepExtents,
                                               up_to_in_use ? engine::ReclaimClass::InUse : engine::ReclaimClass::Ordinary, keep_resume_point != 0);
    out[0] = step.madeProgress; out[1] = step.pending; out[2] = step.evictedState; out[3] = step.reclaimedBytes;
    return 0;
  } catch (...) { return -1; }
}
// mode 0 release extents, 1 keep extents, 2 reuse pages
int ref_cache_reclaim_step(void *facade, int mode, int up_to_in_use, int keep_resume_point, int keep_runway, uint64_t *out) {
  try {
    const engine::CacheReclaimMode modes[3] = {engine::CacheReclaimMode::ReleaseExtents, engine::CacheReclaimMode::KeepExtents, engine::CacheReclaimMode::ReusePages};
    const auto step = FACADE->cache.reclaimOne(modes[mode], up_to_in_use ? engine::ReclaimClass::InUse : engine::ReclaimClass::Ordinary,
                                               keep_resume_point != 0, keep_runway != 0);
    out[0] = step.madeProgress; out[1] = step.pending; out[2] = step.evictedState; out[3] = step.reclaimedBytes;
    return 0;
  } catch (...) { return -1; }
}
// Cache::evictAll: out[2] = made progress, extent bytes returned
int ref_cache_evict_all(void *facade, uint64_t *out) {
  try {
    const auto step = FACADE->cache.evictAll();
    out[0] = step.madeProgress; out[1] = step.reclaimedBytes;
    return 0;
  } catch (...) { return -1; }
}
int ref_cache_reclaim_one_state(void *facade, int checkpoints_only, uint64_t for_block) {
  try { return FACADE->cache.reclaimOneState(checkpoints_only != 0, for_block, false) ? 1 : 0; } catch (...) { return -1; }
}
// What the facade keeps private, read for the comparison (the shim is compiled with -fno-access-control).
// out[8] = block known, page, has tier copy, transferring, matchable, state contained, state resident, state ordinary
int ref_cache_block_info(void *facade, uint64_t block, uint64_t *out) {
  try {
    auto &cache = FACADE->cache;
    for (int i = 0; i < 8; ++i) out[i] = 0;
    if (!cache.kv_.contains(block)) return 0;
    out[0] = 1; out[1] = cache.kv_.page(block); out[2] = cache.kv_.slot(block) != nullptr; out[3] = cache.kv_.transferring(block);
    out[4] = cache.kv_.matchable(block); out[5] = cache.states_.contains(block); out[6] = cache.states_.stateResident(block);
    out[7] = cache.states_.ordinary(block);
    return 0;
  } catch (...) { return -1; }
}
int ref_cache_poll(void *facade) { try { return FACADE->cache.pollTransfers() ? 1 : 0; } catch (...) { return -1; } }
// out[12] = pagesAllocated, pagesFree, pagesActive, pagesPrefix, state entries, state bytes, pinned states,
//           tier blocks, pending pages, demotions, restores, demotions refused; out[12..15] = KV tokens hit, lazy
//           junctions, lost-state misses, pages hashed by probes
void ref_cache_snapshot(void *facade, uint64_t *out) {
  const auto s = FACADE->cache.snapshot();
  out[0] = s.pool.pagesAllocated; out[1] = s.pool.pagesFree; out[2] = s.pool.pagesActive; out[3] = s.pool.pagesPrefix;
  out[4] = s.stateCache.entries; out[5] = s.stateCache.bytes; out[6] = s.stateCache.pinned;
  out[7] = s.kvTier.diskBlocks; out[8] = s.kvTier.pendingPages; out[9] = s.kvTier.demotions; out[10] = s.kvTier.restores;
  out[11] = s.kvTier.demotionsRefused;
  out[12] = s.lookup.kvHitTokens; out[13] = s.lookup.lazyJunctions; out[14] = s.lookup.lostStateMisses; out[15] = s.lookup.probeHashedBlocks;
}
// Cache::adopt on a cache with a persistent tier (with_tier == 2 at creation). KV labels cross as they lie in a slot
// file's records (label i has sizes[i] bytes, back to back); each adopted slot is a fresh slot of the test tier. One
// stored state per (state_blocks[i], state_tokens[i]) names the restore points: the reference takes a chain back only
// for a state. out[4] = states, blocks, bytes, dropped.
int ref_cache_adopt(void *facade, const uint8_t *labels, const uint32_t *sizes, uint32_t count, const uint64_t *state_blocks,
                    const uint32_t *state_tokens, const uint64_t *state_last_used, uint32_t states, uint64_t *out) {
  try {
    std::vector<engine::PersistedKv> blocks;
    test::TestKvTier *tier = FACADE->tier.get();
    for (uint32_t i = 0; i < count; ++i) {
      engine::PersistedKv block;
      block.label.assign(reinterpret_cast<const std::byte *>(labels), reinterpret_cast<const std::byte *>(labels) + sizes[i]);
      block.adopt = [tier] { return tier->adopt(); };
      blocks.push_back(std::move(block));
      labels += sizes[i];
    }
    std::vector<engine::PersistedState> kept;
    for (uint32_t i = 0; i < states; ++i) {
      engine::PersistedState state;
      state.label = engine::encodeLabel(engine::StateLabel{state_blocks[i], state_last_used[i], state_tokens[i], 0});
      state.adopt = [](uint32_t) { return std::make_shared<StoredState>(64); }; // every state is 64 bytes here
      kept.push_back(std::move(state));
    }
    const engine::CacheAdoption result = FACADE->cache.adopt(std::move(blocks), std::move(kept));
    out[0] = result.states; out[1] = result.blocks; out[2] = result.bytes; out[3] = result.dropped;
    return 0;
  } catch (...) { return -1; }
}
// The same with the state labels as they lie in a states' file: `states` StateLabel records of 24 bytes.
int ref_cache_adopt_labelled(void *facade, const uint8_t *labels, const uint32_t *sizes, uint32_t count, const uint8_t *state_labels,
                             uint32_t states, uint64_t *out) {
  try {
    std::vector<engine::PersistedKv> blocks;
    test::TestKvTier *tier = FACADE->tier.get();
    for (uint32_t i = 0; i < count; ++i) {
      engine::PersistedKv block;
      block.label.assign(reinterpret_cast<const std::byte *>(labels), reinterpret_cast<const std::byte *>(labels) + sizes[i]);
      block.adopt = [tier] { return tier->adopt(); };
      blocks.push_back(std::move(block));
      labels += sizes[i];
    }
    std::vector<engine::PersistedState> kept;
    for (uint32_t i = 0; i < states; ++i) {
      engine::PersistedState state;
      const auto *at = reinterpret_cast<const std::byte *>(state_labels) + size_t(i) * sizeof(engine::StateLabel);
      state.label.assign(at, at + sizeof(engine::StateLabel));
      state.adopt = [](uint32_t) { return std::make_shared<StoredState>(64); };
      kept.push_back(std::move(state));
    }
    const engine::CacheAdoption result = FACADE->cache.adopt(std::move(blocks), std::move(kept));
    out[0] = result.states; out[1] = result.blocks; out[2] = result.bytes; out[3] = result.dropped;
    return 0;
  } catch (...) { return -1; }
}
// Cache::relabelStates (what a clean stop does), then the label of every stored state alive, 24 bytes each, with its size.
int ref_cache_state_labels(void *facade, uint8_t *out, uint64_t *sizes, uint32_t capacity) {
  try {
    FACADE->cache.relabelStates();
    uint32_t count = 0;
    for (const StoredState *state : StoredState::alive()) {
      if (state->kept().size() != sizeof(engine::StateLabel)) continue;
      if (count < capacity) { std::memcpy(out + size_t(count) * sizeof(engine::StateLabel), state->kept().data(), sizeof(engine::StateLabel)); sizes[count] = state->bytes(); }
      ++count;
    }
    return int(count);
  } catch (...) { return -1; }
}
// The labels a persistent test tier's slots carry (Cache labels a copy when it lands), 168 bytes each, in no order.
int ref_cache_tier_labels(void *facade, uint8_t *out, uint32_t capacity) {
  try {
    uint32_t count = 0;
    for (const auto &label : FACADE->tier->labels()) {
      if (label.size() != sizeof(engine::KvBlockLabel)) return -2;
      if (count < capacity) std::memcpy(out + size_t(count) * sizeof(engine::KvBlockLabel), label.data(), label.size());
      ++count;
    }
    return int(count);
  } catch (...) { return -1; }
}
#undef FACADE


// ---- the reference's persistent slot file --------------------------------------------------
namespace {
model::SlotFile::Persistence persistence_of(const char *slots, const char *records, const void *tag, uint32_t tag_bytes, uint32_t label_bytes) {
  model::SlotFile::Persistence p;
  p.slots = slots; p.records = records; p.labelBytes = label_bytes;
  p.tag.assign(static_cast<const std::byte *>(tag), static_cast<const std::byte *>(tag) + tag_bytes);
  return p;
}
} // namespace

// Opens (or creates) the pair of files, drops what an earlier process left, and writes `count` slots: payload i
// (payload_bytes each) with label i (label_bytes each), each write waited for, then a flush to the drive and a clean
// seal. Returns the slots written, or -1.
int ref_slotfile_write(const char *slots, const char *records, const void *tag, uint32_t tag_bytes, uint32_t label_bytes,
                       uint64_t slot_bytes, uint32_t count, const uint8_t *payloads, uint64_t payload_bytes, const uint8_t *labels) {
  try {
    auto budget = std::make_shared<model::DiskBudget>(uint64_t(1) << 40);
    model::SlotFile file(slot_bytes, budget, persistence_of(slots, records, tag, tag_bytes, label_bytes));
    file.finishAdoption();
    std::vector<std::shared_ptr<model::SlotFile::Slot>> held;
    int written = 0;
    for (uint32_t i = 0; i < count; ++i) {
      auto slot = file.acquire();
      if (!slot) return -1;
      const auto *bytes = reinterpret_cast<const std::byte *>(payloads + uint64_t(i) * payload_bytes);
      auto operation = file.write(slot, {std::span<const std::byte>(bytes, payload_bytes)}, {});
      if (!operation) return -1;
      const auto *label = reinterpret_cast<const std::byte *>(labels + uint64_t(i) * label_bytes);
      file.label(slot, std::vector<std::byte>(label, label + label_bytes));
      if (!operation->wait()) return -1;
      held.push_back(std::move(slot));
      ++written;
    }
    auto flushed = file.synchronize({});
    if (!flushed || !flushed->wait()) return -1;
    file.seal();
    return written;
  } catch (...) { return -1; }
}

// Opens the pair of files and reports what an earlier process left: per record its slot index, payload size and
// checksum, its label (label_bytes each into labels), and the payload read back through an adopted slot (whose first
// read is checked against the record) into payloads (payload_capacity each); ok[i] = that read succeeded. Returns the
// records found (at most capacity are reported), or -1. The files stay as they were.
int ref_slotfile_read(const char *slots, const char *records, const void *tag, uint32_t tag_bytes, uint32_t label_bytes,
                      uint64_t slot_bytes, uint32_t capacity, uint32_t *indices, uint64_t *payload_bytes, uint32_t *checksums,
                      uint8_t *labels, uint8_t *payloads, uint64_t payload_capacity, uint8_t *ok) {
  try {
    auto budget = std::make_shared<model::DiskBudget>(uint64_t(1) << 40);
    model::SlotFile file(slot_bytes, budget, persistence_of(slots, records, tag, tag_bytes, label_bytes));
    const std::vector<model::SlotRecord> found = file.records();
    std::vector<std::shared_ptr<model::SlotFile::Slot>> held;
    for (const model::SlotRecord &record : found) held.push_back(file.adopt(record));
    file.finishAdoption();
    for (size_t i = 0; i < found.size() && i < capacity; ++i) {
      indices[i] = found[i].index; payload_bytes[i] = found[i].payloadBytes; checksums[i] = found[i].checksum;
      std::memcpy(labels + i * label_bytes, found[i].label.data(), std::min<size_t>(label_bytes, found[i].label.size()));
      auto *destination = reinterpret_cast<std::byte *>(payloads + i * payload_capacity);
      const uint64_t size = std::min<uint64_t>(payload_capacity, found[i].payloadBytes);
      auto operation = file.read(held[i], {std::span<std::byte>(destination, size)}, {});
      ok[i] = operation && operation->wait();
    }
    file.seal();
    return int(found.size());
  } catch (...) { return -1; }
}

} // extern "C"

