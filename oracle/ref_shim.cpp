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
#include "Q8PageFormatReference.hpp"
#include "Fp8PageFormatReference.hpp"
#include "engine/cache/KvPool.hpp"
#include "ops/PagedAttention.hpp"

#include <cstring>
#include <memory>
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

} // extern "C"
