// ref_metal_kernels.cpp — the reference's OWN store, tree-compaction and attention kernels (Metal source), compiled as C++ in place
// from the reference checkout and run on the host: one fiber per Metal thread of a threadgroup, switched at barriers,
// 32 consecutive threads a SIMD group, independent threadgroups on the host's cores. Address spaces and kernel attributes mean nothing on the host;
// everything else — the row decode, the page addressing, the maximum reduction, the quantiser expressions, the nibble
// packing, the copy order of the compaction, the attention tile's page loop with its admission rule, scale folds, online
// softmax, bf16 probabilities and conditional rescale, and the fixed-order merge of the splits — is the reference's
// text (never copied into this repository). The tensor operations the tile calls are stood in for by
// metal_shim/MetalPerformancePrimitives (plain fp32 sums in index order; Metal's fast::exp is std::exp), so attention
// agrees with the Metal kernels up to their arithmetic, not bit for bit.
//
// TEST INFRASTRUCTURE ONLY: built by oracle/Makefile into oracle/_ref/ where the reference checkout is present, used
// by tests/ to pin the checker's stores and compaction against the reference kernels themselves.
#include <ucontext.h>

#include <functional>
#include <stdexcept>
#include <memory>
#include <thread>
#include <vector>

#include "metal/kernels/common/attention_qkv_prepare.h"
#include "metal/kernels/common/paged_attention_tile.h"
#include "metal/kernels/decode/fp8_attention.metal"
#include "metal/kernels/decode/fp8_attention_store.metal"
#include "metal/kernels/decode/paged_attention.metal"
#include "metal/kernels/decode/paged_attention_store.metal"
#include "metal/kernels/prefill/fp8_attention_store.metal"
#include "metal/kernels/prefill/paged_attention.metal"
#include "metal/kernels/prefill/paged_attention_store.metal"

thread_local uint rk_metal_thread_index = 0;

namespace {
constexpr uint kThreads = 256, kSimd = 32;
// One threadgroup in flight: its 256 Metal threads are user-level fibers (ucontext) of ONE host thread, switched at
// barriers only, so a barrier costs a context swap instead of a futex round over 256 host threads, and a threadgroup
// runs deterministically. Independent threadgroups run on as many host threads as the machine has cores.
struct Group {
  enum class State : uint8_t { Ready, AtThreadgroupBarrier, AtSimdBarrier, Done };
  ucontext_t scheduler;
  ucontext_t contexts[kThreads];
  State states[kThreads];
  std::unique_ptr<char[]> stacks;
  static constexpr size_t kStack = 128 * 1024;
  std::function<void(uint)> body; // what fiber t runs
  float floats[kThreads];
  uint words[kThreads];
  float maxima[8]; // the kernels' `threadgroup float maxima[8]`
  // the attention entries' threadgroup scratch, sized for sixteen rows of an eight-head group
  static constexpr uint kRows = 128;
  alignas(16) float scores[kRows * 32];
  alignas(16) bfloat probabilities[2 * kRows * 32];
  float row_max[kRows], row_sum[kRows], previous_scale[kRows];
  std::atomic<uint> rescale{0};
  float weights[RICHENGINE_VERIFY_ATTENTION_MAXIMUM_SPLITS], group_values[8];
  alignas(16) half half_probabilities[kRows * 32];   // the fp8 entries' fp16 probabilities and staged queries
  alignas(16) half staged_queries[kRows / 2 * 256];
  bfloat normalized[256];                            // the QKV-prepare entries' normalised row
  Group() : stacks(new char[kThreads * kStack]) {}
  void run();
};
thread_local Group *group_of_thread = nullptr;
#define index_of_thread rk_metal_thread_index

void fiber_entry() {
  Group &g = *group_of_thread;
  const uint t = index_of_thread;
  g.body(t);
  g.states[t] = Group::State::Done;
  swapcontext(&g.contexts[t], &g.scheduler);
}

// Runs the 256 fibers of one threadgroup to completion: every ready fiber runs until its next barrier; a SIMD-group
// barrier opens when its 32 fibers (those not finished) wait at it, the threadgroup barrier when all of them do.
void Group::run() {
  for (uint t = 0; t < kThreads; ++t) {
    getcontext(&contexts[t]);
    contexts[t].uc_stack.ss_sp = stacks.get() + size_t(t) * kStack;
    contexts[t].uc_stack.ss_size = kStack;
    contexts[t].uc_link = &scheduler;
    makecontext(&contexts[t], fiber_entry, 0);
    states[t] = State::Ready;
  }
  for (;;) {
    uint alive = 0;
    for (uint t = 0; t < kThreads; ++t) {
      if (states[t] == State::Ready) {
        index_of_thread = t;
        swapcontext(&scheduler, &contexts[t]);
      }
      alive += states[t] != State::Done;
    }
    if (!alive) return;
    bool released = false;
    for (uint base = 0; base < kThreads; base += kSimd) {
      uint waiting = 0, others = 0;
      for (uint t = base; t < base + kSimd; ++t) {
        waiting += states[t] == State::AtSimdBarrier;
        others += states[t] == State::AtThreadgroupBarrier || states[t] == State::Ready;
      }
      if (waiting && !others) {
        for (uint t = base; t < base + kSimd; ++t)
          if (states[t] == State::AtSimdBarrier) states[t] = State::Ready;
        released = true;
      }
    }
    if (released) continue;
    for (uint t = 0; t < kThreads; ++t)
      if (states[t] == State::AtSimdBarrier) throw std::logic_error("a SIMD-group barrier some of its threads never reach");
    for (uint t = 0; t < kThreads; ++t)
      if (states[t] == State::AtThreadgroupBarrier) states[t] = State::Ready;
  }
}

void wait_at(Group::State barrier) {
  Group &g = *group_of_thread;
  const uint t = index_of_thread;
  g.states[t] = barrier;
  swapcontext(&g.contexts[t], &g.scheduler);
  index_of_thread = t;
}

// Runs `groups` threadgroups, independent of one another, over the host's cores.
template <typename Body> void dispatch(uint groups, Body body) {
  const uint workers = std::max(1u, std::min(groups, std::thread::hardware_concurrency()));
  std::atomic<uint> next{0};
  std::atomic<bool> failed{false};
  std::vector<std::thread> threads;
  for (uint w = 0; w < workers; ++w)
    threads.emplace_back([&] {
      auto shared = std::make_unique<Group>();
      group_of_thread = shared.get();
      try {
        for (uint g = next.fetch_add(1); g < groups; g = next.fetch_add(1)) {
          shared->body = [&, g](uint t) { body(g, t, t % kSimd, t / kSimd, *shared); };
          shared->run();
        }
      } catch (...) { failed = true; }
    });
  for (std::thread &t : threads) t.join();
  if (failed) throw std::runtime_error("a threadgroup failed");
}
} // namespace

namespace metal {
void threadgroup_barrier(mem_flags) { wait_at(Group::State::AtThreadgroupBarrier); }
void simdgroup_barrier(mem_flags) { wait_at(Group::State::AtSimdBarrier); }
float simd_max(float value) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd;
  g.floats[index_of_thread] = value;
  wait_at(Group::State::AtSimdBarrier);
  float result = g.floats[base];
  for (uint lane = 1; lane < kSimd; ++lane) result = max(result, g.floats[base + lane]);
  wait_at(Group::State::AtSimdBarrier);
  return result;
}
// Metal leaves the order of a SIMD-group sum to the hardware; this one is the xor butterfly 16, 8, 4, 2, 1 (every lane
// ends with the same value), the order the checker fixes too.
float simd_sum(float value) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd, lane = index_of_thread - base;
  for (uint step = kSimd / 2; step != 0; step >>= 1) {
    g.floats[index_of_thread] = value;
    wait_at(Group::State::AtSimdBarrier);
    value += g.floats[base + (lane ^ step)];
    wait_at(Group::State::AtSimdBarrier);
  }
  return value;
}
float simd_shuffle_xor(float value, ushort mask) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd;
  g.floats[index_of_thread] = value;
  wait_at(Group::State::AtSimdBarrier);
  const float result = g.floats[base + ((index_of_thread - base) ^ mask)];
  wait_at(Group::State::AtSimdBarrier);
  return result;
}
uint simd_shuffle_xor(uint value, ushort mask) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd;
  g.words[index_of_thread] = value;
  wait_at(Group::State::AtSimdBarrier);
  const uint result = g.words[base + ((index_of_thread - base) ^ mask)];
  wait_at(Group::State::AtSimdBarrier);
  return result;
}
} // namespace metal

namespace {
template <typename Element>
void verify_store(const bfloat *keys, const bfloat *values, const RichKvPage *const *tables, const RichChunkedPrefillParams *params, uint lanes) {
  const uint groups = lanes * 2 * params[0].chunk_tokens * 4;
  dispatch(groups, [&](uint group, uint thread, uint lane, uint simd, Group &shared) {
    richengine_store_verify_phase<4, Element>(keys, values, tables[0], tables[1], tables[2], tables[3], params, shared.maxima, group, thread, lane, simd);
  });
}
template <typename Element>
void chunk_store(const bfloat *keys, const bfloat *values, const RichKvPage *table, const RichChunkedPrefillParams &params) {
  dispatch(2 * params.chunk_tokens * 4, [&](uint group, uint thread, uint lane, uint simd, Group &shared) {
    richengine_store_chunk_phase<4, Element>(keys, values, table, params, shared.maxima, group, thread, lane, simd);
  });
}
void verify_store_fp8(const bfloat *keys, const bfloat *values, const RichKvPage *const *tables, const RichChunkedPrefillParams *params, uint lanes) {
  dispatch(lanes * 2 * RICHENGINE_TARGET_VERIFY_ROWS * 4, [&](uint group, uint thread, uint lane, uint simd, Group &shared) {
    richengine_store_fp8_verify_phase<4>(keys, values, tables[0], tables[1], tables[2], tables[3], params, shared.maxima, group, thread, lane, simd);
  });
}
void chunk_store_fp8(const bfloat *keys, const bfloat *values, const RichKvPage *table, const RichChunkedPrefillParams &params) {
  dispatch(2 * params.chunk_tokens * 4, [&](uint group, uint thread, uint lane, uint simd, Group &shared) {
    richengine_store_fp8_chunk_phase<4>(keys, values, table, params, shared.maxima, group, thread, lane, simd);
  });
}
// The fp8 chain verify entry (decode/fp8_attention.metal:8-50, a macro body restated here: placement as the other
// entries'), then the shared reduce phase.
void verify_attention_fp8(bfloat *queries, const RichKvPage *const *tables, const RichVerifyAttentionParams *params, uint lanes,
                          float *partials, float *statistics, bfloat *output) {
  constexpr uint KVHeads = 4, Q = 6, D = 256, Rows = RICHENGINE_TARGET_VERIFY_ROWS, M = Rows * Q;
  constexpr ulong group_stride = ulong(RICHENGINE_VERIFY_CHUNK_STRIDE) * Q * D;
  uint most_splits = 0;
  for (uint lane = 0; lane < lanes; ++lane) most_splits = max(most_splits, params[lane].split_count);
  dispatch(lanes * most_splits * KVHeads, [&](uint group, uint thread, uint, uint, Group &shared) {
    const uint kv_head = group % KVHeads, split = group / KVHeads % most_splits, lane = group / (KVHeads * most_splits);
    const RichVerifyAttentionParams &p = params[lane];
    if (!richengine_verify_attention_contract_valid(p) || split >= p.split_count) return;
    richengine_paged_attention_tile_fp8<KVHeads, Q, Rows, D>(
        queries + (ulong(lane) * KVHeads + kv_head) * group_stride, tables[lane], p.kv, kv_head, p.committed_tokens, Rows, p.split_count, split,
        partials, statistics, (ulong(lane) * KVHeads + kv_head) * p.slot_splits + split, shared.scores, shared.half_probabilities,
        shared.row_max, shared.row_sum, shared.previous_scale, &shared.rescale, shared.staged_queries, thread, p.score_scale);
  });
  dispatch(lanes * M * KVHeads, [&](uint group, uint thread, uint, uint, Group &shared) {
    const uint3 at{group % KVHeads, group / KVHeads % M, group / (KVHeads * M)};
    richengine_verify_attention_reduce_phase<KVHeads, Q, D>(partials, statistics, output, params, at, thread, shared.weights, shared.group_values);
  });
}
// The step before the path (decode/attention_qkv.metal:6-32, whose offsets per lane are restated here, over the
// reference's full_qkv_storage_phase): per (lane, row) the packed projection row becomes the stagings the store and
// the attention read. 24 query heads with their gates, 4 KV heads, fp32 or bf16 norm weights.
template <typename Weight>
void qkv_prepare(const bfloat *qkv, const Weight *q_norm, const Weight *k_norm, const float *rope_cos, const float *rope_sin,
                 bfloat *queries, bfloat *keys, bfloat *values, uint lanes, uint rows) {
  constexpr uint QHeads = 24, KHeads = 4, HeadDim = 256, RotaryPairs = 32, Stride = RICHENGINE_VERIFY_CHUNK_STRIDE;
  constexpr uint PackedStride = QHeads * 2 * HeadDim + 2 * KHeads * HeadDim;
  const uint tasks = rows * (QHeads + KHeads);
  dispatch(lanes * tasks, [&](uint group, uint thread, uint lane, uint simd, Group &shared) {
    const uint batch = group / tasks, task = group % tasks;
    const ulong kv_lane_stride = ulong(KHeads) * Stride * HeadDim;
    FullPrefillParams lane_params{rows, Stride};
    full_qkv_storage_phase<QHeads, KHeads>(qkv + ulong(batch) * rows * PackedStride, q_norm, k_norm, rope_cos + ulong(batch) * rows * RotaryPairs,
                                           rope_sin + ulong(batch) * rows * RotaryPairs, queries + ulong(batch) * QHeads * Stride * HeadDim,
                                           keys + ulong(batch) * kv_lane_stride, values + ulong(batch) * kv_lane_stride, lane_params,
                                           shared.group_values, shared.normalized, task, thread, lane, simd);
  });
}
template <typename Element>
void tree_compact(const RichKvPage *const *tables, const RichChunkedPrefillParams *params, const uint *path, const uint *count, uint lanes) {
  dispatch(lanes * 4, [&](uint group, uint thread, uint, uint, Group &) {
    richengine_compact_verify_tree_phase<4, Element>(tables[0], tables[1], tables[2], tables[3], params, path, count, group, thread);
  });
}
// One verify step as the reference dispatches it (decode/paged_attention.metal): its own tile placement
// (richengine_verify_attention_tile_at) for a threadgroup per (KV head, split, lane), the tile, then its own reduce phase
// for a threadgroup per (KV head, fused row, lane). Rows = 8: the chain entries (every tile processes all eight rows,
// the causal limit per row); Rows = 16: the tree entries (the lane's active rows and its ancestor masks). Four KV heads
// of Q query heads each, head dimension 256. With gate buffers the chain's reduce is its reduce/gate phase.
template <typename Element, uint Rows, uint Q>
void verify_attention(bfloat *queries, const RichKvPage *const *tables, const RichVerifyAttentionParams *params, uint lanes,
                      const uint *row_masks, float *partials, float *statistics, bfloat *output, const bfloat *packed_qkv = nullptr,
                      bfloat *hidden = nullptr) {
  constexpr uint KVHeads = 4, D = 256, M = Rows * Q;
  constexpr bool chain = Rows == RICHENGINE_TARGET_VERIFY_ROWS;
  uint most_splits = 0;
  for (uint lane = 0; lane < lanes; ++lane) most_splits = max(most_splits, params[lane].split_count);
  dispatch(lanes * most_splits * KVHeads, [&](uint group, uint thread, uint, uint, Group &shared) {
    const uint3 at{group % KVHeads, group / KVHeads % most_splits, group / (KVHeads * most_splits)};
    const RichVerifyTile tile = richengine_verify_attention_tile_at<KVHeads, Q, D>(queries, tables[0], tables[1], tables[2], tables[3], params, at);
    if (!tile.active) return;
    const uint *masks = chain ? nullptr : row_masks + ulong(at.z) * params[at.z].row_capacity;
    richengine_paged_attention_tile<KVHeads, Q, Rows, Element, D>(
        tile.queries, tile.page_table, params[at.z].kv, tile.kv_head, tile.committed_tokens, chain ? Rows : tile.active_rows, tile.splits,
        tile.split, partials, statistics, tile.slot, masks, params[at.z].score_scale, shared.scores, shared.probabilities,
        shared.row_max, shared.row_sum, shared.previous_scale, &shared.rescale, thread);
  });
  dispatch(lanes * M * KVHeads, [&](uint group, uint thread, uint, uint, Group &shared) {
    const uint3 at{group % KVHeads, group / KVHeads % M, group / (KVHeads * M)};
    if constexpr (chain) {
      if (hidden) richengine_verify_attention_reduce_gate_phase<KVHeads, Q>(partials, statistics, output, packed_qkv, hidden, params, at, thread, shared.weights, shared.group_values);
      else richengine_verify_attention_reduce_phase<KVHeads, Q, D>(partials, statistics, output, params, at, thread, shared.weights, shared.group_values);
    } else {
      richengine_verify_tree_attention_reduce_phase<KVHeads, Q, D>(partials, statistics, output, params, at, thread, shared.weights, shared.group_values);
    }
  });
}

// A prefill chunk as the reference dispatches it (prefill/paged_attention.metal): its own split and reduce phases
// place the tiles; a threadgroup per (KV head, tile, split), then one per (KV head, fused row, tile). One row is the
// plain decode step.
template <typename Element>
void prefill_attention(bfloat *queries, const RichKvPage *table, const RichPrefillAttentionParams &params, float *partials, float *statistics, bfloat *output) {
  constexpr uint KVHeads = 4, Q = 6, M = RICHENGINE_PREFILL_ATTENTION_TILE_ROWS * Q;
  const uint tiles = (params.rows + RICHENGINE_PREFILL_ATTENTION_TILE_ROWS - 1) / RICHENGINE_PREFILL_ATTENTION_TILE_ROWS;
  dispatch(KVHeads * tiles * params.split_count, [&](uint group, uint thread, uint, uint, Group &shared) {
    const uint3 at{group % KVHeads, group / KVHeads % tiles, group / (KVHeads * tiles)};
    richengine_prefill_attention_split_phase<KVHeads, Q, Element>(queries, partials, statistics, table, params, shared.scores, shared.probabilities,
                                                                  shared.row_max, shared.row_sum, shared.previous_scale, &shared.rescale, at, thread);
  });
  dispatch(KVHeads * M * tiles, [&](uint group, uint thread, uint, uint, Group &shared) {
    const uint3 at{group % KVHeads, group / KVHeads % M, group / (KVHeads * M)};
    richengine_prefill_attention_reduce_phase<KVHeads, Q>(partials, statistics, output, params, at, thread, shared.weights, shared.group_values);
  });
}
} // namespace

extern "C" {
// A prefill chunk (or, with one row, a decode step) of one sequence: queries and output are [4][chunk_stride][6][256]
// bf16; partials [(tile*4 + head)*split_count + split][48][256] fp32, statistics [..][48]{max, sum}.
int ref_metal_attention_prefill(uint32_t format, void *queries, const uint64_t *table, const void *params, float *partials, float *statistics, void *output) {
  try {
    auto *q = static_cast<bfloat *>(queries), *o = static_cast<bfloat *>(output);
    const auto *t = reinterpret_cast<const RichKvPage *>(table);
    const auto &p = *static_cast<const RichPrefillAttentionParams *>(params);
    if (format == 1) prefill_attention<int8_t>(q, t, p, partials, statistics, o);
    else if (format == 2) prefill_attention<bfloat>(q, t, p, partials, statistics, o);
    else if (format == 3) prefill_attention<RichKvPacked4>(q, t, p, partials, statistics, o);
    else return -1;
    return 0;
  } catch (...) { return -1; }
}
// A verify step over `lanes` lanes (at most four) of four KV heads with `group` (6 or 4) query heads each: queries and
// output are [lane][4][32][group][256] bf16; partials [(lane*4 + head)*slot_splits + split][rows*group][256] fp32 and
// statistics [..][rows*group]{max, sum}, as the kernels lay them out. rows = 8 runs the chain entries, 16 the tree
// entries (row_masks [lane][row_capacity]).
int ref_metal_qkv_prepare(const void *qkv, const void *q_norm, const void *k_norm, int norm_f32, const float *rope_cos, const float *rope_sin,
                          void *queries, void *keys, void *values, uint32_t lanes, uint32_t rows) {
  try {
    const auto *packed = static_cast<const bfloat *>(qkv);
    auto *q = static_cast<bfloat *>(queries), *k = static_cast<bfloat *>(keys), *v = static_cast<bfloat *>(values);
    if (norm_f32) qkv_prepare(packed, static_cast<const float *>(q_norm), static_cast<const float *>(k_norm), rope_cos, rope_sin, q, k, v, lanes, rows);
    else qkv_prepare(packed, static_cast<const bfloat *>(q_norm), static_cast<const bfloat *>(k_norm), rope_cos, rope_sin, q, k, v, lanes, rows);
    return 0;
  } catch (...) { return -1; }
}
// packed_qkv and hidden (both or neither; chain entries of six heads only) bind the gate buffers: the merge is then the
// reduce/gate phase, which also writes hidden [lane][8][24][256] bf16 from the gate values of packed_qkv [lane][8][stride].
int ref_metal_attention_verify(uint32_t format, uint32_t rows, uint32_t group, void *queries, const uint64_t *const *tables, const void *params,
                               uint32_t lanes, const uint32_t *row_masks, float *partials, float *statistics, void *output,
                               const void *packed_qkv, void *hidden) {
  try {
    auto *q = static_cast<bfloat *>(queries), *o = static_cast<bfloat *>(output);
    const auto *t = reinterpret_cast<const RichKvPage *const *>(tables);
    const auto *p = static_cast<const RichVerifyAttentionParams *>(params);
    const auto run = [&](auto element, auto row_count, auto heads) {
      verify_attention<typename decltype(element)::type, decltype(row_count)::value, decltype(heads)::value>(
          q, t, p, lanes, row_masks, partials, statistics, o, static_cast<const bfloat *>(packed_qkv), static_cast<bfloat *>(hidden));
    };
    const auto with_shape = [&](auto element) {
      if (rows == 8 && group == 6) run(element, std::integral_constant<uint, 8>{}, std::integral_constant<uint, 6>{});
      else if (rows == 8 && group == 4) run(element, std::integral_constant<uint, 8>{}, std::integral_constant<uint, 4>{});
      else if (rows == 16 && group == 6) run(element, std::integral_constant<uint, 16>{}, std::integral_constant<uint, 6>{});
      else if (rows == 16 && group == 4) run(element, std::integral_constant<uint, 16>{}, std::integral_constant<uint, 4>{});
      else throw 0;
    };
    if (format == 4 && rows == 8 && group == 6 && !hidden) { verify_attention_fp8(q, t, p, lanes, partials, statistics, o); return 0; }
    if (format == 1) with_shape(std::type_identity<int8_t>{});
    else if (format == 2) with_shape(std::type_identity<bfloat>{});
    else if (format == 3) with_shape(std::type_identity<RichKvPacked4>{});
    else return -1;
    return 0;
  } catch (...) { return -1; }
}
// format: 1 int8, 2 bf16, 3 int4, 4 fp8 e4m3 (kv::Format). Four KV heads, head dimension 256. tables: four page-table pointers
// (unused lanes may repeat the first). params: `lanes` RichChunkedPrefillParams.
int ref_metal_store_verify(uint32_t format, const void *keys, const void *values, const uint64_t *const *tables, const void *params, uint32_t lanes) {
  try {
    const auto *k = static_cast<const bfloat *>(keys), *v = static_cast<const bfloat *>(values);
    const auto *t = reinterpret_cast<const RichKvPage *const *>(tables);
    const auto *p = static_cast<const RichChunkedPrefillParams *>(params);
    if (format == 4) verify_store_fp8(k, v, t, p, lanes);
    else if (format == 1) verify_store<int8_t>(k, v, t, p, lanes);
    else if (format == 2) verify_store<bfloat>(k, v, t, p, lanes);
    else if (format == 3) verify_store<RichKvPacked4>(k, v, t, p, lanes);
    else return -1;
    return 0;
  } catch (...) { return -1; }
}
int ref_metal_store_chunk(uint32_t format, const void *keys, const void *values, const uint64_t *table, const void *params) {
  try {
    const auto *k = static_cast<const bfloat *>(keys), *v = static_cast<const bfloat *>(values);
    const auto *t = reinterpret_cast<const RichKvPage *>(table);
    const auto &p = *static_cast<const RichChunkedPrefillParams *>(params);
    if (format == 4) chunk_store_fp8(k, v, t, p);
    else if (format == 1) chunk_store<int8_t>(k, v, t, p);
    else if (format == 2) chunk_store<bfloat>(k, v, t, p);
    else if (format == 3) chunk_store<RichKvPacked4>(k, v, t, p);
    else return -1;
    return 0;
  } catch (...) { return -1; }
}
int ref_metal_tree_compact(uint32_t format, const uint64_t *const *tables, const void *params, const uint32_t *path, const uint32_t *count, uint32_t lanes) {
  try {
    const auto *t = reinterpret_cast<const RichKvPage *const *>(tables);
    const auto *p = static_cast<const RichChunkedPrefillParams *>(params);
    if (format == 1) tree_compact<int8_t>(t, p, path, count, lanes);
    else if (format == 2) tree_compact<bfloat>(t, p, path, count, lanes);
    else if (format == 3) tree_compact<RichKvPacked4>(t, p, path, count, lanes);
    else return -1;
    return 0;
  } catch (...) { return -1; }
}
}
