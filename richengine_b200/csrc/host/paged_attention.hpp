// paged_attention.hpp — the operator layer: plans, parameter factories and the store / attention /
// compaction encoders, mirroring ops::PagedAttention (runtime/ops/PagedAttention.hpp:199-324,
// PagedAttention.cpp:200-573). The reference appends dispatches to a command graph; on CUDA an
// encoder call launches on the caller's stream through the C ABI. Validation happens before the
// first launch, so a refused call encodes nothing.
#pragma once

#include "../../../include/richkv.h"
#include "kv_layout.hpp"

#include <cstdint>
#include <span>
#include <string>
#include <vector>

namespace rkb::ops {

struct DispatchSize { uint64_t x = 1, y = 1, z = 1; };
struct AttentionWorkspace { uint64_t partialsBytes = 0, statisticsBytes = 0; };

inline constexpr uint32_t kVerifyRows = RK_VERIFY_ROWS;
inline constexpr uint32_t kVerifySplits = 32, kVerifyPagesPerSplit = 16;

// One lane's split count: one split per 16 visible pages, at least 32, at most 128
// (PagedAttention.hpp:54-63).
constexpr uint32_t verifyAttentionSplits(uint32_t committedTokens, uint32_t rows = kVerifyRows) noexcept {
  const uint64_t pages = (uint64_t(committedTokens) + rows + kv::kPageTokens - 1) / kv::kPageTokens;
  const uint64_t scaled = (pages + kVerifyPagesPerSplit - 1) / kVerifyPagesPerSplit;
  return uint32_t(std::min<uint64_t>(std::max<uint64_t>(kVerifySplits, scaled), RK_VERIFY_MAX_SPLITS));
}
constexpr uint32_t prefillAttentionTiles(uint32_t rows) noexcept { return (rows + RK_PREFILL_TILE_ROWS - 1) / RK_PREFILL_TILE_ROWS; }
// Empty when valid, else the reference's tag (PagedAttention.hpp:75-95).
std::string_view chunkedPrefillValidationError(const rk_chunk_params &params) noexcept;

struct PrefillAttentionPlan {
  kv::Format format;
  uint32_t rows = 0, splits = 0;
  AttentionWorkspace workspace;
  std::string splitPipeline, reducePipeline;
  DispatchSize splitGroups, reduceGroups, reduceThreads;
  float scoreScale = 0.0f;
};

struct VerifyAttentionPlan {
  kv::Format format;
  uint32_t lanes = 0;
  std::vector<uint32_t> laneSplits;
  uint32_t splits = 0;
  AttentionWorkspace workspace;
  std::string splitPipeline, reducePipeline, storePipeline;
  DispatchSize splitGroups, reduceGroups, storeGroups;
  uint32_t rowCapacity = 0;
  float scoreScale = 0.0f;
  // Row capacity 1 on int4, int8 or fp8 pages runs the streaming decode kernel instead of split + reduce.
  bool streamingDecode = false;
  rk_decode_plan decode{};
  // Row capacity 8 or 16 on int4 pages runs the tcgen05 split kernel; laneSplits / splits / splitGroups then
  // hold its partition (one CTA per (lane, head, split), the SMs filled once) instead of the reference's.
  bool tensorCoreWindow = false;
};

struct PagedVerifyBuffers {
  void *chunkKeys = nullptr, *chunkValues = nullptr, *queries = nullptr, *output = nullptr;
  float *partials = nullptr, *statistics = nullptr;
  uint32_t *descriptors = nullptr;                   // streaming decode only
  uint32_t *status = nullptr;                        // tcgen05 window kernel only: one zeroed device word
  const rk_page_entry *const *pageTables = nullptr;  // device array, one table address per lane
  const uint32_t *treeMasks = nullptr;
  uint64_t partialsBytes = 0, statisticsBytes = 0;   // sizes of the scratch actually bound
};

class PagedAttention final {
public:
  static PrefillAttentionPlan prefillPlan(uint32_t rows, uint32_t queryHeads, kv::Layout layout);
  // historyTokens: each lane's committed tokens before its rows. rowCapacity 0 selects the
  // reference's 8 (chain) or 16 (tree); 1 is the plain decode. ctas sizes the streaming grid (0 = SMs).
  static uint32_t windowSplits(uint32_t lanes, uint32_t kvHeads, uint32_t visibleTokens, uint32_t ctas);
  static VerifyAttentionPlan verifyPlan(uint32_t lanes, uint32_t queryHeads, kv::Layout layout,
                                        std::span<const uint32_t> historyTokens, bool tree = false,
                                        uint32_t rowCapacity = 0, uint32_t ctas = 148);
  static AttentionWorkspace prefillWorkspace(uint32_t maximumRows, uint32_t queryHeads, kv::Layout layout);
  static AttentionWorkspace verifyWorkspace(uint32_t lanes, uint32_t queryHeads, kv::Layout layout);

  static rk_chunk_params prefillParams(uint64_t logicalPosition, uint32_t chunkTokens, uint32_t chunkStride, uint32_t pageTableEntries);
  static rk_chunk_params verifyParams(uint64_t logicalPosition, uint32_t pageTableEntries);
  static rk_chunk_params verifyTreeParams(uint64_t logicalPosition, uint32_t pageTableEntries);

  static void addPrefillStore(void *stream, rk_kv_layer layer, const void *chunkKeys, const void *chunkValues,
                              const rk_page_entry *pageTable, const rk_chunk_params &params, kv::Layout layout);
  static void addPrefill(void *stream, rk_kv_layer layer, const void *queries, void *output, float *partials,
                         float *statistics, uint64_t partialsBytes, uint64_t statisticsBytes,
                         const rk_page_entry *pageTable, const rk_chunk_params &chunk, const PrefillAttentionPlan &plan,
                         uint32_t queryHeads, kv::Layout layout,
                         // the pool's window and one zeroed device word select the tcgen05 kernel for the tiles
                         const void *window = nullptr, uint32_t *status = nullptr);
  // deviceChunks / deviceAttention: the lanes' parameter blocks in device memory (uploaded once per step).
  static void addVerify(void *stream, rk_kv_layer layer, const PagedVerifyBuffers &buffers,
                        const rk_chunk_params *deviceChunks, const rk_verify_params *deviceAttention,
                        const VerifyAttentionPlan &plan, uint32_t queryHeads, kv::Layout layout, const void *window = nullptr);
  static void addVerifyTreeCompact(void *stream, rk_kv_layer layer, const rk_page_entry *const *pageTables,
                                   const uint32_t *retainedPath, const uint32_t *retained,
                                   const rk_chunk_params *deviceChunks, uint32_t lanes, kv::Layout layout);
};

} // namespace rkb::ops
