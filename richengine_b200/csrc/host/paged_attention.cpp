#include "paged_attention.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <limits>
#include <stdexcept>

namespace rkb::ops {
namespace {

// The kernel family's geometry tags (PagedAttention.cpp:37-145). Only the 256-wide layouts of the
// 27B family have kernels here; the names of the others are kept so plans can be compared.
std::string_view attentionSuffix(const kv::Layout &layout, uint32_t queryHeads) {
  if (layout.headDimension == 256 && layout.kvHeads == 4) {
    if (queryHeads == 24) return "";
    if (queryHeads == 16) return "_kv4_g4";
  }
  if (layout.headDimension == 256 && layout.kvHeads == 2 && queryHeads == 16) return "_kv2_g8";
  if (layout.headDimension == 128 && layout.kvHeads == 2 && queryHeads == 16) return "_hd128";
  if (layout.headDimension == 64 && layout.kvHeads == 8 && queryHeads == 32) return "_hd64";
  if (layout.headDimension == 64 && layout.kvHeads == 8 && queryHeads == 40) return "_k8q5d64";
  if (layout.headDimension == 128 && layout.kvHeads == 8 && queryHeads == 32) return "_k8q4d128";
  throw std::invalid_argument("unsupported attention layout");
}
std::string_view storageSuffix(const kv::Layout &layout) {
  if (layout.headDimension == 256 && layout.kvHeads == 4) return "";
  if (layout.headDimension == 256 && layout.kvHeads == 2) return "_kv2_g8";
  if (layout.headDimension == 128 && layout.kvHeads == 2) return "_hd128";
  if (layout.headDimension == 64 && layout.kvHeads == 8) return "_hd64";
  if (layout.headDimension == 128 && layout.kvHeads == 8) return "_k8d128";
  throw std::invalid_argument("unsupported attention layout");
}
const char *formatTag(kv::Format format) noexcept {
  switch (format) {
  case kv::Format::Int8: return "q8";
  case kv::Format::Int4: return "int4";
  case kv::Format::BFloat16: return "bf16";
  case kv::Format::Float8E4M3: return "fp8";
  }
  return "";
}
constexpr uint32_t prefillSplits(uint32_t tiles) { return std::clamp(RK_PREFILL_MAX_SPLITS / tiles, 1u, RK_PREFILL_MAX_SPLITS); }
AttentionWorkspace workspaceFor(uint64_t fusedRows, uint32_t headDimension) {
  return {fusedRows * headDimension * sizeof(float), fusedRows * 2 * sizeof(float)};
}
void check(int status) {
  if (status == RK_OK) return;
  if (status == RK_ERR_INVALID || status == RK_ERR_UNSUPPORTED) throw std::invalid_argument(rk_last_error());
  throw std::runtime_error(rk_last_error());
}
uint32_t formatCode(kv::Format f) { return static_cast<uint32_t>(f); }

} // namespace

std::string_view chunkedPrefillValidationError(const rk_chunk_params &p) noexcept {
  if (!p.chunk_tokens || p.chunk_tokens > RK_PREFILL_TOKEN_BUDGET) return "chunk_tokens_out_of_range";
  if (uint64_t(p.committed_tokens) + p.chunk_tokens > RK_MAX_PHYSICAL_TOKENS) return "context_out_of_range";
  if (p.chunk_stride < p.chunk_tokens || p.chunk_stride > RK_PREFILL_TOKEN_BUDGET || p.chunk_stride % kv::kPageTokens) return "chunk_stride_invalid";
  if (p.page_table_entries < rk_pages_for(p.committed_tokens + p.chunk_tokens)) return "page_table_too_short";
  return {};
}

AttentionWorkspace PagedAttention::prefillWorkspace(uint32_t maximumRows, uint32_t queryHeads, kv::Layout layout) {
  (void)attentionSuffix(layout, queryHeads);
  if (!maximumRows || maximumRows > RK_PREFILL_TOKEN_BUDGET) throw std::invalid_argument("invalid attention workspace rows");
  uint64_t slots = 0; // allocation-time bound for every shorter sequence
  for (uint32_t tiles = 1; tiles <= prefillAttentionTiles(maximumRows); ++tiles) slots = std::max(slots, uint64_t(tiles) * prefillSplits(tiles));
  return workspaceFor(slots * RK_PREFILL_TILE_ROWS * queryHeads, layout.headDimension);
}

AttentionWorkspace PagedAttention::verifyWorkspace(uint32_t lanes, uint32_t queryHeads, kv::Layout layout) {
  (void)attentionSuffix(layout, queryHeads);
  if (!lanes) throw std::invalid_argument("invalid attention workspace batch width");
  return workspaceFor(uint64_t(lanes) * RK_TREE_NODES * RK_VERIFY_MAX_SPLITS * queryHeads, layout.headDimension);
}

PrefillAttentionPlan PagedAttention::prefillPlan(uint32_t rows, uint32_t queryHeads, kv::Layout layout) {
  const std::string suffix(attentionSuffix(layout, queryHeads));
  if (!rows || rows > RK_PREFILL_TOKEN_BUDGET || !kv::validFormat(layout.format)) throw std::invalid_argument("invalid paged prefill attention geometry");
  const uint32_t tiles = prefillAttentionTiles(rows), splits = prefillSplits(tiles);
  const uint32_t fusedRows = RK_PREFILL_TILE_ROWS * (queryHeads / layout.kvHeads);
  PrefillAttentionPlan plan;
  plan.format = layout.format;
  plan.rows = rows;
  plan.splits = splits;
  plan.workspace = workspaceFor(uint64_t(tiles) * splits * layout.kvHeads * fusedRows, layout.headDimension);
  plan.splitPipeline = std::string("prefill_attention_") + formatTag(layout.format) + "_split" + suffix;
  plan.reducePipeline = "prefill_attention_reduce" + suffix;
  plan.splitGroups = {layout.kvHeads, tiles, splits};
  plan.reduceGroups = {layout.kvHeads, fusedRows, tiles};
  plan.reduceThreads = {layout.headDimension, 1, 1};
  plan.scoreScale = layout.scoreScale;
  return plan;
}

// Multiprocessors of the current device; 0 where there is none (a host without a GPU keeps the reference plan).
static uint32_t deviceMultiprocessors() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return uint32_t(sms);
}

// Split count of one lane for the tcgen05 window kernel: (lanes x heads x splits) CTAs fill the SMs once, a
// split holds an even number of pages (whole 64-token groups) unless it is the lane's only one.
uint32_t PagedAttention::windowSplits(uint32_t lanes, uint32_t kvHeads, uint32_t visibleTokens, uint32_t ctas) {
  const uint32_t pages = rk_pages_for(visibleTokens);
  uint32_t splits = std::clamp<uint32_t>(ctas / std::max<uint32_t>(1, lanes * kvHeads), 1, RK_VERIFY_MAX_SPLITS);
  splits = std::min(splits, std::max<uint32_t>(1, (pages + 1) / 2));
  uint32_t perSplit = (pages + splits - 1) / splits;
  if (splits > 1 && (perSplit & 1u)) ++perSplit;
  return std::max<uint32_t>(1, (pages + perSplit - 1) / perSplit);
}

VerifyAttentionPlan PagedAttention::verifyPlan(uint32_t lanes, uint32_t queryHeads, kv::Layout layout,
                                               std::span<const uint32_t> historyTokens, bool tree, uint32_t rowCapacity, uint32_t ctas) {
  const std::string suffix(attentionSuffix(layout, queryHeads));
  if (!kv::validFormat(layout.format)) throw std::invalid_argument("paged attention requires a kv format");
  if (tree && layout.format == kv::Format::Float8E4M3) throw std::invalid_argument("tree verify has no fp8 kernels");
  if (!lanes || historyTokens.size() != lanes) throw std::invalid_argument("verify lane count is out of range");
  const uint32_t rows = rowCapacity ? rowCapacity : (tree ? RK_TREE_NODES : kVerifyRows);
  if (rows != 1 && rows != kVerifyRows && rows != RK_TREE_NODES) throw std::invalid_argument("row capacity is 1, 8 or 16");
  const uint32_t liveRows = rowCapacity ? rowCapacity : (tree ? RK_TREE_NODES - 1 : kVerifyRows);
  VerifyAttentionPlan plan;
  plan.format = layout.format;
  plan.lanes = lanes;
  plan.laneSplits.resize(lanes);
  for (uint32_t lane = 0; lane < lanes; ++lane) {
    if (uint64_t(historyTokens[lane]) + liveRows > kv::kMaximumPhysicalTokens) throw std::invalid_argument("verify attention history exceeds physical context");
    plan.laneSplits[lane] = verifyAttentionSplits(historyTokens[lane], liveRows);
    plan.splits = std::max(plan.splits, plan.laneSplits[lane]);
  }
  plan.workspace = workspaceFor(uint64_t(lanes) * rows * RK_VERIFY_MAX_SPLITS * queryHeads, layout.headDimension);
  const char *stem = tree ? "verify_tree_attention" : "verify_attention";
  plan.splitPipeline = std::string(stem) + "_" + formatTag(layout.format) + "_split" + suffix;
  plan.reducePipeline = std::string(stem) + "_reduce" + suffix;
  plan.storePipeline = std::string("verify_attention_") + formatTag(layout.format) + "_store" + std::string(storageSuffix(layout));
  plan.splitGroups = {layout.kvHeads, plan.splits, lanes};
  plan.reduceGroups = {layout.kvHeads, uint64_t(rows) * (queryHeads / layout.kvHeads), lanes};
  plan.storeGroups = {uint64_t(lanes) * 2 * liveRows * layout.kvHeads, 1, 1};
  plan.rowCapacity = rows;
  plan.scoreScale = layout.scoreScale;
  if (rows == 1 &&
      rk_decode_plan_make(formatCode(layout.format), layout.kvHeads, queryHeads, layout.headDimension, lanes, ctas, &plan.decode) == RK_OK) {
    plan.streamingDecode = true;
    plan.workspace = {plan.decode.partials_bytes, plan.decode.statistics_bytes};
  }
  if ((rows == kVerifyRows || rows == RK_TREE_NODES) && layout.format == kv::Format::Int4 && layout.kvHeads == 4 &&
      queryHeads == 24 && layout.headDimension == 256) {
    if (!ctas) ctas = deviceMultiprocessors();
    if (ctas) {
      plan.tensorCoreWindow = true;
      plan.splits = 0;
      for (uint32_t lane = 0; lane < lanes; ++lane) {
        plan.laneSplits[lane] = windowSplits(lanes, layout.kvHeads, historyTokens[lane] + liveRows, ctas);
        plan.splits = std::max(plan.splits, plan.laneSplits[lane]);
      }
      plan.splitGroups = {layout.kvHeads, plan.splits, lanes};
    }
  }
  return plan;
}

rk_chunk_params PagedAttention::prefillParams(uint64_t logicalPosition, uint32_t chunkTokens, uint32_t chunkStride, uint32_t pageTableEntries) {
  if (logicalPosition > std::numeric_limits<uint32_t>::max()) throw std::overflow_error("KV logical position exceeds kernel ABI");
  rk_chunk_params params{uint32_t(logicalPosition), chunkTokens, chunkStride, pageTableEntries, {0, 0}};
  if (const std::string_view error = chunkedPrefillValidationError(params); !error.empty()) throw std::invalid_argument(std::string(error));
  return params;
}
rk_chunk_params PagedAttention::verifyParams(uint64_t logicalPosition, uint32_t pageTableEntries) {
  return prefillParams(logicalPosition, kVerifyRows, RK_VERIFY_CHUNK_STRIDE, pageTableEntries);
}
rk_chunk_params PagedAttention::verifyTreeParams(uint64_t logicalPosition, uint32_t pageTableEntries) {
  return prefillParams(logicalPosition, RK_TREE_NODES - 1, RK_VERIFY_CHUNK_STRIDE, pageTableEntries);
}

void PagedAttention::addPrefillStore(void *stream, rk_kv_layer layer, const void *chunkKeys, const void *chunkValues,
                                     const rk_page_entry *pageTable, const rk_chunk_params &params, kv::Layout layout) {
  (void)storageSuffix(layout);
  rk_chunk_params chunk = params;
  chunk.kv = layer;
  if (const std::string_view error = chunkedPrefillValidationError(chunk); !error.empty()) throw std::invalid_argument(std::string(error));
  check(rk_store_chunk(formatCode(layout.format), layout.kvHeads, layout.headDimension, chunkKeys, chunkValues, pageTable, &chunk, stream));
}

void PagedAttention::addPrefill(void *stream, rk_kv_layer layer, const void *queries, void *output, float *partials, float *statistics,
                                uint64_t partialsBytes, uint64_t statisticsBytes, const rk_page_entry *pageTable,
                                const rk_chunk_params &chunk, const PrefillAttentionPlan &plan, uint32_t queryHeads, kv::Layout layout,
                                const void *window, uint32_t *status) {
  if (chunk.chunk_tokens != plan.rows) throw std::invalid_argument("prefill attention rows do not match plan");
  if (const std::string_view error = chunkedPrefillValidationError(chunk); !error.empty()) throw std::invalid_argument(std::string(error));
  if (partialsBytes < plan.workspace.partialsBytes || statisticsBytes < plan.workspace.statisticsBytes)
    throw std::invalid_argument("prefill attention scratch is smaller than its bound");
  if (queries == output) throw std::invalid_argument("queries and output must not alias");
  const rk_prefill_params attention{chunk.committed_tokens, chunk.chunk_tokens, chunk.chunk_stride, chunk.page_table_entries, layer, plan.splits, plan.scoreScale};
  if (window && status && layout.kvHeads == 4 && queryHeads == 24 && layout.headDimension == 256)
    check(rk_attention_prefill_split_tc(window, formatCode(layout.format), layout.kvHeads, queryHeads, layout.headDimension, queries, partials,
                                        statistics, pageTable, &attention, status, stream));
  else
    check(rk_attention_prefill_split(formatCode(layout.format), layout.kvHeads, queryHeads, layout.headDimension, queries, partials, statistics, pageTable, &attention, stream));
  check(rk_attention_prefill_reduce(layout.kvHeads, queryHeads, layout.headDimension, partials, statistics, output, nullptr, &attention, stream));
}

void PagedAttention::addVerify(void *stream, rk_kv_layer layer, const PagedVerifyBuffers &b, const rk_chunk_params *deviceChunks,
                               const rk_verify_params *deviceAttention, const VerifyAttentionPlan &plan, uint32_t queryHeads,
                               kv::Layout layout, const void *window) {
  if (!b.pageTables || !deviceChunks || !deviceAttention) throw std::invalid_argument("invalid paged verify batch");
  if (b.partialsBytes < plan.workspace.partialsBytes || b.statisticsBytes < plan.workspace.statisticsBytes)
    throw std::invalid_argument("verify attention scratch is smaller than its bound");
  if (b.queries == b.output) throw std::invalid_argument("queries and output must not alias");
  const bool tree = plan.rowCapacity > kVerifyRows;
  if (tree && !b.treeMasks) throw std::invalid_argument("tree verify requires its ancestor masks");
  if (plan.streamingDecode && (!window || !b.descriptors)) throw std::invalid_argument("streaming decode needs the pool window and its descriptors");
  if (plan.tensorCoreWindow && !plan.streamingDecode && (!window || !b.status))
    throw std::invalid_argument("the window kernel needs the pool window and a status word");
  if (!b.chunkKeys || !b.chunkValues || !b.queries || !b.output || !b.partials || !b.statistics) throw std::invalid_argument("invalid paged verify batch");
  // every check is done: from here on the call launches
  const uint32_t format = formatCode(layout.format);
  check(rk_store_verify(format, layout.kvHeads, layout.headDimension, plan.lanes, std::min<uint32_t>(plan.rowCapacity, RK_TREE_NODES),
                        b.chunkKeys, b.chunkValues, b.pageTables, deviceChunks, layer, stream));
  if (plan.streamingDecode) {
    check(rk_attention_decode(window, &plan.decode, format, b.queries, b.output, nullptr, b.partials, b.statistics, b.descriptors,
                              b.pageTables, deviceAttention, layer, stream));
    return;
  }
  if (plan.tensorCoreWindow) {
    check(rk_attention_verify_split_tc(window, format, layout.kvHeads, queryHeads, layout.headDimension, plan.lanes, plan.rowCapacity,
                                       plan.splits, b.queries, b.partials, b.statistics, b.pageTables, tree ? b.treeMasks : nullptr,
                                       deviceAttention, layer, b.status, stream));
  } else {
    check(rk_attention_verify_split(format, layout.kvHeads, queryHeads, layout.headDimension, plan.lanes, plan.rowCapacity, plan.splits,
                                    b.queries, b.partials, b.statistics, b.pageTables, tree ? b.treeMasks : nullptr, deviceAttention, layer, stream));
  }
  check(rk_attention_verify_reduce(layout.kvHeads, queryHeads, layout.headDimension, plan.lanes, plan.rowCapacity, b.partials, b.statistics,
                                   b.output, nullptr, deviceAttention, stream));
}

void PagedAttention::addVerifyTreeCompact(void *stream, rk_kv_layer layer, const rk_page_entry *const *pageTables, const uint32_t *retainedPath,
                                          const uint32_t *retained, const rk_chunk_params *deviceChunks, uint32_t lanes, kv::Layout layout) {
  if (!lanes || !pageTables || !deviceChunks) throw std::invalid_argument("invalid tree verify compact batch");
  if (layout.format == kv::Format::Float8E4M3) throw std::invalid_argument("tree verify has no fp8 kernels");
  check(rk_tree_compact(formatCode(layout.format), layout.kvHeads, layout.headDimension, lanes, pageTables, deviceChunks, layer, retainedPath, retained, stream));
}

} // namespace rkb::ops
