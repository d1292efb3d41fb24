// ref_metal_store.cpp — the reference's OWN store and tree-compaction kernels (Metal source), compiled as C++ in place
// from the reference checkout and run on host threads: one std::thread per Metal thread of a threadgroup, barriers as
// std::barrier, 32 consecutive threads a SIMD group. Address spaces and kernel attributes mean nothing on the host;
// everything else — the row decode, the page addressing, the maximum reduction, the quantiser expressions, the nibble
// packing, the copy order of the compaction — is the reference's text (never copied into this repository).
//
// TEST INFRASTRUCTURE ONLY: built by oracle/Makefile into oracle/_ref/ where the reference checkout is present, used
// by tests/ to pin the checker's stores and compaction against the reference kernels themselves.
#include <barrier>
#include <memory>
#include <thread>
#include <vector>

#include "metal/kernels/decode/paged_attention_store.metal"
#include "metal/kernels/prefill/paged_attention_store.metal"

namespace {
constexpr uint kThreads = 256, kSimd = 32;
struct Group {
  std::barrier<> all{kThreads};
  std::vector<std::unique_ptr<std::barrier<>>> simd;
  float floats[kThreads];
  uint words[kThreads];
  float maxima[8]; // the kernels' `threadgroup float maxima[8]`
  Group() { for (uint i = 0; i < kThreads / kSimd; ++i) simd.push_back(std::make_unique<std::barrier<>>(kSimd)); }
};
thread_local Group *group_of_thread = nullptr;
thread_local uint index_of_thread = 0;

// Runs `groups` threadgroups one after another on 256 persistent host threads.
template <typename Body> void dispatch(uint groups, Body body) {
  Group shared;
  std::vector<std::thread> threads;
  for (uint t = 0; t < kThreads; ++t)
    threads.emplace_back([&, t] {
      group_of_thread = &shared;
      index_of_thread = t;
      for (uint g = 0; g < groups; ++g) {
        body(g, t, t % kSimd, t / kSimd, shared.maxima);
        shared.all.arrive_and_wait(); // the next threadgroup starts with this one's memory settled
      }
    });
  for (std::thread &t : threads) t.join();
}
} // namespace

namespace metal {
void threadgroup_barrier(mem_flags) { group_of_thread->all.arrive_and_wait(); }
void simdgroup_barrier(mem_flags) { group_of_thread->simd[index_of_thread / kSimd]->arrive_and_wait(); }
float simd_max(float value) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd;
  g.floats[index_of_thread] = value;
  g.simd[base / kSimd]->arrive_and_wait();
  float result = g.floats[base];
  for (uint lane = 1; lane < kSimd; ++lane) result = max(result, g.floats[base + lane]);
  g.simd[base / kSimd]->arrive_and_wait();
  return result;
}
float simd_sum(float value) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd;
  g.floats[index_of_thread] = value;
  g.simd[base / kSimd]->arrive_and_wait();
  float result = 0.0f;
  for (uint lane = 0; lane < kSimd; ++lane) result += g.floats[base + lane];
  g.simd[base / kSimd]->arrive_and_wait();
  return result;
}
uint simd_shuffle_xor(uint value, ushort mask) {
  Group &g = *group_of_thread;
  const uint base = index_of_thread / kSimd * kSimd;
  g.words[index_of_thread] = value;
  g.simd[base / kSimd]->arrive_and_wait();
  const uint result = g.words[base + ((index_of_thread - base) ^ mask)];
  g.simd[base / kSimd]->arrive_and_wait();
  return result;
}
} // namespace metal

namespace {
template <typename Element>
void verify_store(const bfloat *keys, const bfloat *values, const RichKvPage *const *tables, const RichChunkedPrefillParams *params, uint lanes) {
  const uint groups = lanes * 2 * params[0].chunk_tokens * 4;
  dispatch(groups, [&](uint group, uint thread, uint lane, uint simd, float *maxima) {
    richengine_store_verify_phase<4, Element>(keys, values, tables[0], tables[1], tables[2], tables[3], params, maxima, group, thread, lane, simd);
  });
}
template <typename Element>
void chunk_store(const bfloat *keys, const bfloat *values, const RichKvPage *table, const RichChunkedPrefillParams &params) {
  dispatch(2 * params.chunk_tokens * 4, [&](uint group, uint thread, uint lane, uint simd, float *maxima) {
    richengine_store_chunk_phase<4, Element>(keys, values, table, params, maxima, group, thread, lane, simd);
  });
}
template <typename Element>
void tree_compact(const RichKvPage *const *tables, const RichChunkedPrefillParams *params, const uint *path, const uint *count, uint lanes) {
  dispatch(lanes * 4, [&](uint group, uint thread, uint, uint, float *) {
    richengine_compact_verify_tree_phase<4, Element>(tables[0], tables[1], tables[2], tables[3], params, path, count, group, thread);
  });
}
} // namespace

extern "C" {
// format: 1 int8, 2 bf16, 3 int4 (kv::Format). Four KV heads, head dimension 256. tables: four page-table pointers
// (unused lanes may repeat the first). params: `lanes` RichChunkedPrefillParams.
int ref_metal_store_verify(uint32_t format, const void *keys, const void *values, const uint64_t *const *tables, const void *params, uint32_t lanes) {
  try {
    const auto *k = static_cast<const bfloat *>(keys), *v = static_cast<const bfloat *>(values);
    const auto *t = reinterpret_cast<const RichKvPage *const *>(tables);
    const auto *p = static_cast<const RichChunkedPrefillParams *>(params);
    if (format == 1) verify_store<int8_t>(k, v, t, p, lanes);
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
    if (format == 1) chunk_store<int8_t>(k, v, t, p);
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
